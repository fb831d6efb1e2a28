/* Forwarding header: code written against the reference's include layout (nocta/optim/sgd.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_OPTIM_SGD_H
#define NOCTA_FWD_OPTIM_SGD_H
#include "../nocta.h"
#endif
