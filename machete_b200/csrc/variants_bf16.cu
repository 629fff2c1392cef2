// Kernel variants: bf16 weights, up to 8 activation rows: the decode step (plain, traced, tensor parallel), the bare matvec, head dim 128.
// One translation unit per group so that the groups compile in parallel.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {1, 0, MK_F_AT64 | MK_F_TOP1, mk::mk_persistent_kernel<1, 0, MK_F_AT64 | MK_F_TOP1>},
    {1, 0, MK_F_AT64 | MK_F_TOP1 | MK_F_TRACE, mk::mk_persistent_kernel<1, 0, MK_F_AT64 | MK_F_TOP1 | MK_F_TRACE>},
    {1, 0, MK_F_AT64 | MK_F_TOP1 | MK_F_AR, mk::mk_persistent_kernel<1, 0, MK_F_AT64 | MK_F_TOP1 | MK_F_AR>},
    {1, 0, MK_F_TOP1, mk::mk_persistent_kernel<1, 0, MK_F_TOP1>},
    {1, 0, MK_F_AT128 | MK_F_TOP1, mk::mk_persistent_kernel<1, 0, MK_F_AT128 | MK_F_TOP1>},
};

extern "C" const mk_variant* mk_variants_bf16(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
