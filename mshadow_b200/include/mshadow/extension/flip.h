/* Kept so that `#include <mshadow/extension/flip.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_FLIP_H_
#define MSHADOW_EXTENSION_COMPAT_FLIP_H_
#include "./remap.h"
#endif
