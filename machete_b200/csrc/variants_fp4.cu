// Kernel variants: NVFP4 weights, up to 8 activation rows.
// One translation unit per group so that the groups compile in parallel.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1, mk::mk_persistent_kernel<1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1>},
    {1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_TRACE, mk::mk_persistent_kernel<1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_TRACE>},
    {1, 2, MK_F_TOP1, mk::mk_persistent_kernel<1, 2, MK_F_TOP1>},
    {1, 2, MK_F_AT64 | MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_EW, mk::mk_persistent_kernel<1, 2, MK_F_AT64 | MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_EW>},
};

extern "C" const mk_variant* mk_variants_fp4(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
