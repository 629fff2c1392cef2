// Kernel variants: NVFP4 weights, 9-16 and 17-32 activation rows.
// One translation unit per group so that the groups compile in parallel.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {2, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1, mk::mk_persistent_kernel<2, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1>},
    {4, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1, mk::mk_persistent_kernel<4, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1>},
    {2, 2, MK_F_TOP1, mk::mk_persistent_kernel<2, 2, MK_F_TOP1>},
    {4, 2, MK_F_TOP1, mk::mk_persistent_kernel<4, 2, MK_F_TOP1>},
};

extern "C" const mk_variant* mk_variants_fp4_wide(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
