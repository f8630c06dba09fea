/* See hip_runtime.h in this directory: host-only stand-in, test infrastructure. */
#include "hip_runtime.h"
