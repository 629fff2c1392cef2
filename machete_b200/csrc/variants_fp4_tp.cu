// Kernel variants: NVFP4 weights with the in-kernel all-reduce (tensor parallel).
// One translation unit per group so that the groups compile in parallel.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR, mk::mk_persistent_kernel<1, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR>},
    {2, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR, mk::mk_persistent_kernel<2, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR>},
    {4, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR, mk::mk_persistent_kernel<4, 2, MK_F_AT128 | MK_F_QKNORM | MK_F_TOP1 | MK_F_AR>},
};

extern "C" const mk_variant* mk_variants_fp4_tp(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
