/* Kept so that `#include <mshadow/extension/slice.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SLICE_H_
#define MSHADOW_EXTENSION_COMPAT_SLICE_H_
#include "./remap.h"
#endif
