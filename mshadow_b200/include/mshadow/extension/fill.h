/* Kept so that `#include <mshadow/extension/fill.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_FILL_H_
#define MSHADOW_EXTENSION_COMPAT_FILL_H_
#include "./select.h"
#endif
