// Drop-in for ruy/ruy.h: the ruy API over libruy_b200.so (see ruy_b200_shim.h).
#include "ruy/ruy_b200_shim.h"
