/* Kept so that `#include <mshadow/extension/swapaxis.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_SWAPAXIS_H_
#define MSHADOW_EXTENSION_COMPAT_SWAPAXIS_H_
#include "./remap.h"
#endif
