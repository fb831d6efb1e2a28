/* Forwarding header: code written against the reference's include layout (nocta/ops/loss.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_OPS_LOSS_H
#define NOCTA_FWD_OPS_LOSS_H
#include "../nocta.h"
#endif
