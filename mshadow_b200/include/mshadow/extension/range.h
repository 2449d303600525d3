/* Kept so that `#include <mshadow/extension/range.h>` keeps working; see axis.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_RANGE_H_
#define MSHADOW_EXTENSION_COMPAT_RANGE_H_
#include "./axis.h"
#endif
