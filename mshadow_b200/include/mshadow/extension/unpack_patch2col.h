/* Kept so that `#include <mshadow/extension/unpack_patch2col.h>` keeps working; see patch.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_UNPACK_PATCH2COL_H_
#define MSHADOW_EXTENSION_COMPAT_UNPACK_PATCH2COL_H_
#include "./patch.h"
#endif
