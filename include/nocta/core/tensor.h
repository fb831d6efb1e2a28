/* Forwarding header: code written against the reference's include layout (nocta/core/tensor.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_CORE_TENSOR_H
#define NOCTA_FWD_CORE_TENSOR_H
#include "../nocta.h"
#endif
