/* Forwarding header: code written against the reference's include layout (nocta/core/serialize.h)
 * finds the same declarations in the single public header of this library. */
#ifndef NOCTA_FWD_CORE_SERIALIZE_H
#define NOCTA_FWD_CORE_SERIALIZE_H
#include "../nocta.h"
#endif
