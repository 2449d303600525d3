/* Kept so that `#include <mshadow/extension/pad.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_PAD_H_
#define MSHADOW_EXTENSION_COMPAT_PAD_H_
#include "./remap.h"
#endif
