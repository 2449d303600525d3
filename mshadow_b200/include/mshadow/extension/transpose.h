/* Kept so that `#include <mshadow/extension/transpose.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_TRANSPOSE_H_
#define MSHADOW_EXTENSION_COMPAT_TRANSPOSE_H_
#include "./remap.h"
#endif
