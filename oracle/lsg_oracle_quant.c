/* FP8 / NVFP4 activation-quantizer oracles (test infrastructure only). */
#include <stdint.h>
