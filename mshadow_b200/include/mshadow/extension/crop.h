/* Kept so that `#include <mshadow/extension/crop.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_CROP_H_
#define MSHADOW_EXTENSION_COMPAT_CROP_H_
#include "./remap.h"
#endif
