/* Kept so that `#include <mshadow/extension/broadcast_with_axis.h>` keeps working; see axis.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_BROADCAST_WITH_AXIS_H_
#define MSHADOW_EXTENSION_COMPAT_BROADCAST_WITH_AXIS_H_
#include "./axis.h"
#endif
