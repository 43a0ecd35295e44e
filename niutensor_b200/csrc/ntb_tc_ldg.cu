/*
 * Instantiations of the single-CTA tensor-core kernel whose operands are fetched by loader
 * warps with ordinary loads (see the loader branch of GemmTcKernel): the route for matrices
 * whose base address or row pitch is not a multiple of 16 bytes, which TMA cannot address.
 * NiuTensor's memory pools hand out tensors back to back with no alignment beyond the
 * element size (source/tensor/XMem.cpp:668-686), so an activation that follows an
 * odd-sized index tensor in a pool starts on a 4-byte (fp32) or 2-byte (fp16) boundary.
 */
#include "ntb_tc_single.cuh"

namespace ntb {

int LaunchLdgKernel(const TcGroup & grp, int mode, int dtC, bool oldc, int smCount, cudaStream_t stream)
{
#define NTB_LDG(MD, W, ST, T) (oldc ? LaunchOne<MD, W, ST, 1, T, true, true>(grp, smCount, stream) \
                                    : LaunchOne<MD, W, ST, 1, T, false, true>(grp, smCount, stream))
    if (mode == 0)
        return dtC == NTB_X_FLOAT16 ? NTB_LDG(0, 128, 5, __half) : NTB_LDG(0, 128, 5, float);
    return NTB_LDG(1, 128, 3, float);
#undef NTB_LDG
}

}
