/* Kept so that `#include <mshadow/extension/take_grad.h>` keeps working; see select.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_TAKE_GRAD_H_
#define MSHADOW_EXTENSION_COMPAT_TAKE_GRAD_H_
#include "./select.h"
#endif
