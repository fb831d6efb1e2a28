/* Forwarding header: code written against the reference's include layout (nocta/nn/module.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_NN_MODULE_H
#define NOCTA_FWD_NN_MODULE_H
#include "../nocta.h"
#endif
