/*
 * Extension expressions of the engine.  Included by tensor.h; user code may also include it
 * directly, as with dmlc/mshadow's mshadow/extension.h.
 */
#ifndef MSHADOW_EXTENSION_H_
#define MSHADOW_EXTENSION_H_
#include "./engine/check.h"
#include "./extension/broadcast.h"
#include "./extension/reduceto1d.h"
#include "./extension/pooling.h"
#include "./extension/remap.h"
#include "./extension/select.h"
#include "./extension/patch.h"
#include "./extension/axis.h"
#include "./extension/complex.h"
#include "./extension/lrn.h"
#endif  // MSHADOW_EXTENSION_H_
