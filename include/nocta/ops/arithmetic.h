/* Forwarding header: code written against the reference's include layout (nocta/ops/arithmetic.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_OPS_ARITHMETIC_H
#define NOCTA_FWD_OPS_ARITHMETIC_H
#include "../nocta.h"
#endif
