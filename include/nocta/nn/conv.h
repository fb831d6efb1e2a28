/* Forwarding header: code written against the reference's include layout (nocta/nn/conv.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_NN_CONV_H
#define NOCTA_FWD_NN_CONV_H
#include "../nocta.h"
#endif
