// Kernel variants for programs without a matvec op (attention alone, row-wise ops): with no matvec code
// in the kernel the split-KV attention at head dim 128 keeps its accumulators in registers.
#include "kernel.cuh"

using namespace mk;

static const mk_variant kVariants[] = {
    {-1, 0, MK_F_AT128, mk::mk_persistent_kernel<-1, 0, MK_F_AT128>},
    {-1, 0, MK_F_AT64, mk::mk_persistent_kernel<-1, 0, MK_F_AT64>},
    {-1, 0, MK_F_AT64 | MK_F_AT128 | MK_F_QKNORM | MK_F_EW | MK_F_COMBINE,
     mk::mk_persistent_kernel<-1, 0, MK_F_AT64 | MK_F_AT128 | MK_F_QKNORM | MK_F_EW | MK_F_COMBINE>},
};

extern "C" const mk_variant* mk_variants_attn(int* n) {
  *n = (int)(sizeof(kVariants) / sizeof(kVariants[0]));
  return kVariants;
}
