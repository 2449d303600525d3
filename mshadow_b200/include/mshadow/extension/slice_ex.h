/* Kept so that `#include <mshadow/extension/slice_ex.h>` keeps working; see axis.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SLICE_EX_H_
#define MSHADOW_EXTENSION_COMPAT_SLICE_EX_H_
#include "./axis.h"
#endif
