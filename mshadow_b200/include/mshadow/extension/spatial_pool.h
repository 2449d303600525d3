/* Kept so that `#include <mshadow/extension/spatial_pool.h>` keeps working; see pooling.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SPATIAL_POOL_H_
#define MSHADOW_EXTENSION_COMPAT_SPATIAL_POOL_H_
#include "./pooling.h"
#endif
