// Kernel variants: the kernels that run any program (with and without the event trace) and the attention-only kernel.
// One translation unit per group so that the groups compile in parallel.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {0, -1, MK_F_ALL, mk::mk_persistent_kernel<0, -1, MK_F_ALL>},
    {0, -1, MK_F_ALL & ~MK_F_TRACE, mk::mk_persistent_kernel<0, -1, MK_F_ALL & ~MK_F_TRACE>},
    {0, -1, MK_F_AT64 | MK_F_AT128 | MK_F_COMBINE, mk::mk_persistent_kernel<0, -1, MK_F_AT64 | MK_F_AT128 | MK_F_COMBINE>},
};

extern "C" const mk_variant* mk_variants_generic(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
