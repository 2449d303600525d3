/* Kept so that `#include <mshadow/extension/channel_pool.h>` keeps working; see pooling.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_CHANNEL_POOL_H_
#define MSHADOW_EXTENSION_COMPAT_CHANNEL_POOL_H_
#include "./pooling.h"
#endif
