/* Forwarding header: code written against the reference's include layout (nocta/ops/reduction.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_OPS_REDUCTION_H
#define NOCTA_FWD_OPS_REDUCTION_H
#include "../nocta.h"
#endif
