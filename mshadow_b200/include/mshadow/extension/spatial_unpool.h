/* Kept so that `#include <mshadow/extension/spatial_unpool.h>` keeps working; see pooling.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SPATIAL_UNPOOL_H_
#define MSHADOW_EXTENSION_COMPAT_SPATIAL_UNPOOL_H_
#include "./pooling.h"
#endif
