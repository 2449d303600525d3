/* Kept so that `#include <mshadow/extension/channel_unpool.h>` keeps working; see pooling.h. */
#ifndef MSHADOW_EXTENSION_COMPAT_CHANNEL_UNPOOL_H_
#define MSHADOW_EXTENSION_COMPAT_CHANNEL_UNPOOL_H_
#include "./pooling.h"
#endif
