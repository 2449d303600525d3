/* Kept so that `#include <mshadow/extension/choose.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_CHOOSE_H_
#define MSHADOW_EXTENSION_COMPAT_CHOOSE_H_
#include "./select.h"
#endif
