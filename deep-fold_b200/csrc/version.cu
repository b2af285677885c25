#include "chr_gpu.h"

#ifndef CHR_BUILD_TAG
#define CHR_BUILD_TAG "dev"
#endif

extern "C" const char *chr_nf4_version(void) { return "chr_nf4 sm_100a " CHR_BUILD_TAG; }
