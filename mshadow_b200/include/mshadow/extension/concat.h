/* Kept so that `#include <mshadow/extension/concat.h>` keeps working; see remap.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_CONCAT_H_
#define MSHADOW_EXTENSION_COMPAT_CONCAT_H_
#include "./remap.h"
#endif
