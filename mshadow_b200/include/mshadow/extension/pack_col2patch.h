/* Kept so that `#include <mshadow/extension/pack_col2patch.h>` keeps working; see patch.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_PACK_COL2PATCH_H_
#define MSHADOW_EXTENSION_COMPAT_PACK_COL2PATCH_H_
#include "./patch.h"
#endif
