/* Kept so that `#include <mshadow/extension/reshape.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_RESHAPE_H_
#define MSHADOW_EXTENSION_COMPAT_RESHAPE_H_
#include "./remap.h"
#endif
