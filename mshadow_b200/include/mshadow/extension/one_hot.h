/* Kept so that `#include <mshadow/extension/one_hot.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_ONE_HOT_H_
#define MSHADOW_EXTENSION_COMPAT_ONE_HOT_H_
#include "./select.h"
#endif
