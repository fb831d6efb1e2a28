/* Forwarding header: code written against the reference's include layout (nocta/autograd/node.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_AUTOGRAD_NODE_H
#define NOCTA_FWD_AUTOGRAD_NODE_H
#include "../nocta.h"
#endif
