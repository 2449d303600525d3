/* Kept so that `#include <mshadow/extension/mask.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_MASK_H_
#define MSHADOW_EXTENSION_COMPAT_MASK_H_
#include "./select.h"
#endif
