/* Kept so that `#include <mshadow/extension/spatial_upsampling_nearest.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SPATIAL_UPSAMPLING_NEAREST_H_
#define MSHADOW_EXTENSION_COMPAT_SPATIAL_UPSAMPLING_NEAREST_H_
#include "./select.h"
#endif
