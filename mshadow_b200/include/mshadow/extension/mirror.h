/* Kept so that `#include <mshadow/extension/mirror.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_MIRROR_H_
#define MSHADOW_EXTENSION_COMPAT_MIRROR_H_
#include "./remap.h"
#endif
