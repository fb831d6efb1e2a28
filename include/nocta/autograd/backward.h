/* Forwarding header: code written against the reference's include layout (nocta/autograd/backward.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_AUTOGRAD_BACKWARD_H
#define NOCTA_FWD_AUTOGRAD_BACKWARD_H
#include "../nocta.h"
#endif
