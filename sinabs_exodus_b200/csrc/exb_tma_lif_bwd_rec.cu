// The same backward with v_mem rebuilt from checkpoints and the forward input (see exb_tma_lif_bwd.cuh, REC).
#include "exb_tma_lif_bwd.cuh"

namespace exb {

cudaError_t launch_lif_backward_ckpt_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used)
{
    *used = false;
    if (!a.ckpt || !a.input || a.v_mem || a.gv || a.surr || surr_kind == EXB_SURR_GENERIC) return cudaSuccess;
    if (!eligible(a.B, a.T, a.M) || !aligned16(a.grad_input) || !aligned16(a.ckpt)) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_lif_bwd<EXB_RESET_SUBTRACT, true>(a, surr_kind, s, used)
                                            : surr_lif_bwd<EXB_RESET_TO_VALUE, true>(a, surr_kind, s, used);
}

cudaError_t set_wait_limit_lif_bwd_rec(unsigned int polls) { return set_wait_limit_here(polls); }

// Status word of this translation unit (see read_device_status).
cudaError_t read_device_status_lif_bwd_rec(cudaStream_t s, unsigned int *out)
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
