// TMA-staged fused reverse-time EXODUS backward (time-major layout) and its launchers.
#include "exb_tma_lif_bwd.cuh"

namespace exb {

cudaError_t launch_lif_backward_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used)
{
    *used = false;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.grad_input)) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_lif_bwd<EXB_RESET_SUBTRACT, false>(a, surr_kind, s, used)
                                            : surr_lif_bwd<EXB_RESET_TO_VALUE, false>(a, surr_kind, s, used);
}

cudaError_t set_wait_limit_lif_bwd(unsigned int polls) { return set_wait_limit_here(polls); }

// Status word of this translation unit (see read_device_status).
cudaError_t read_device_status_lif_bwd(cudaStream_t s, unsigned int *out)
{
    static const unsigned int zero = 0;
    cudaError_t e = cudaMemcpyFromSymbolAsync(out, g_exb_status, sizeof(unsigned int), 0, cudaMemcpyDeviceToHost, s);
    if (e != cudaSuccess) return e;
    e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return e;
    if (*out) e = cudaMemcpyToSymbolAsync(g_exb_status, &zero, sizeof(unsigned int), 0, cudaMemcpyHostToDevice, s);
    return e;
}

}  // namespace exb
