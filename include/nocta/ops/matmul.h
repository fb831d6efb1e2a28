/* Forwarding header: code written against the reference's include layout (nocta/ops/matmul.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_OPS_MATMUL_H
#define NOCTA_FWD_OPS_MATMUL_H
#include "../nocta.h"
#endif
