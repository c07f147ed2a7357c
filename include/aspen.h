/* Drop-in name: programs written against the ASPEN reference include "aspen.h".
 * Everything is declared in aspen_b200.h. */
#ifndef ASPEN_H_FORWARD_
#define ASPEN_H_FORWARD_
#include "aspen_b200.h"
#endif
