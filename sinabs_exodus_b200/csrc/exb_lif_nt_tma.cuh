// [N,T] layout, TMA-staged forward spike scan.
//
// The [N,T] layout (the reference's: one row per neuron, time contiguous) asks each neuron's thread
// for consecutive time steps of its own row.  Here a CTA owns 128 rows and walks time in chunks of 32
// steps, moved by TMA as boxes of 128-byte row pieces with the 128-byte swizzle, which is exactly the
// bank-conflict-free tile the threads want (granule g of shared-memory row s at position g ^ (s & 7)).
// A producer warp streams the input boxes through a ring of stages (mbarriers, bounded waits); the four
// consumer warps -- one thread per row -- run the recurrence over the 32 steps of a stage, overwrite the
// stage with the membrane potential and fill a spike tile beside it, and hand both to TMA stores (bulk
// async group), which clip at the end of a row.
//
// Row classes.  A box row should be one whole 128-byte line of global memory, or every piece ends in
// partial sectors (measured at T = 300 with boxes cut at fixed time steps: 4.12 TB/s against 4.47 for the
// cp.async variant, whose chunks follow each row's own lines).  Row n starts n*T floats into the tensor,
// so its position inside a line repeats with period p = 32 / gcd(T mod 32, 32) rows (p <= 8 when
// T % 4 == 0).  The tensor is therefore described to TMA as [N/p][p][T], and a CTA owns 128 rows of ONE
// class j (rows j, j+p, j+2p, ...): they all start at the same position a_j inside their lines, a box of
// [32 steps x 1 class x 32 rows] placed at time coordinate 32k - a_j consists of whole lines, and the CTA
// needs exactly ceil((T + a_j) / 32) chunks.  A load may start at a negative time coordinate (the fill is
// ignored), a store may not: the first chunk of a class with a_j > 0 is stored by the warps themselves.
// T % 32 == 0 is the case p = 1.
//
// Stages of 32 steps, four of them (80 KB per CTA, two CTAs per SM) measured best at T = 320: 5.95 TB/s
// (cp.async variant 5.36); 64 steps x 2 stages 5.81, 32 x 6 (one CTA per SM) 3.75.  On 1 183 744 rows:
// T = 304 (two classes) 5.62 TB/s against 5.10 for the cp.async variant, T = 300 (eight classes) 5.21 against
// 4.46.  (CTAs that mix the classes -- 16-row boxes, every CTA as many chunks as its latest class -- reached
// 4.73 at T = 300; plain 2-D boxes for T % 32 == 0 are no faster than this code with one class.)
// Included by exb_tma_kernels.cu (shares its status word).
#pragma once

#include "exb_nt_tma_common.cuh"

namespace exb {

struct NttMaps {
    CUtensorMap in, spikes, v_mem;
};

// Recurrence of one thread's row over the 32 steps of a stage row: reads the input granules of `tx`, leaves the
// membrane potential there and the spikes in `ts`.  GUARD: the row ends inside this chunk (steps >= T are skipped).
// The two cases are separate code so that the common one carries no per-step predicate.
template <int RESET, bool GUARD>
__device__ __forceinline__ void ntt_chunk(float *tx, float *ts, int sw, int tb, int T, float &v, float &af,
                                          const Neuron &q, const SpikeCfg &cfg, SpikeTotal &cnt)
{
    // the next granule is read before this one's results are written (no shared-memory round trip per granule)
    float4 xn = *reinterpret_cast<const float4 *>(tx + ((0 ^ sw) << 2));
#pragma unroll(GUARD ? 1 : 8)
    for (int g = 0; g < 8; ++g) {
        const int o = (g ^ sw) << 2;
        const float4 x4 = xn;
        if (g < 7) xn = *reinterpret_cast<const float4 *>(tx + (((g + 1) ^ sw) << 2));
        float x[4] = {x4.x, x4.y, x4.z, x4.w};
        float s4[4], u4[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            if (!GUARD || tb + 4 * g + e < T) lif_step<RESET>(v, af, x[e], q, cfg, cnt);
            s4[e] = af;
            u4[e] = v;
        }
        *reinterpret_cast<float4 *>(ts + o) = make_float4(s4[0], s4[1], s4[2], s4[3]);
        *reinterpret_cast<float4 *>(tx + o) = make_float4(u4[0], u4[1], u4[2], u4[3]);
    }
}

// lp: log2 of the number of row classes p; a_base: position (floats) of row 0 inside its 128-byte line, the same
// for the three tensors.  A CTA owns 128 rows of ONE class j = blockIdx.x % p (rows j + p*i, i from
// 128 * (blockIdx.x / p) on): its rows all start `a` floats into their lines, so the whole CTA walks the same time
// window per chunk and needs exactly ceil((T + a) / 32) chunks.
template <int RESET>
__global__ void __launch_bounds__((NTT_WARPS + 1) * 32, 2)
lif_fwd_nt_tma_kernel(const __grid_constant__ NttMaps maps, const LifFwdArgs A, const int nstages, const int lp,
                      const int a_base)
{
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle works on 1 KB atoms: every box must start on one
    float *stages = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    float *spk = stages + (size_t)nstages * NTT_STAGE;                 // one spike stage, a quarter per warp
    Ring *ring = reinterpret_cast<Ring *>(spk + NTT_STAGE);
    ring_init(ring, nstages, NTT_WARPS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M;
    const int T = (int)A.T;
    const int cls = (int)(blockIdx.x & ((1u << lp) - 1u));        // this CTA's class
    const int blk = (int)(blockIdx.x >> lp);                      // its block of 128 rows of that class
    const int a = (a_base + cls * (T & 31)) & 31;                 // (j + p*i) * T = j * T modulo 32 floats
    const int r0 = blk * NTT_ROWS;                                           // first row, counted inside the class
    const int nchunks = (T + a + NTT_BOX_T - 1) / NTT_BOX_T;

    if (warp == NTT_WARPS) {
        if (lane == 0) {
            int s = 0;
            uint32_t par = 0u;
            int k = 0;
            for (; k < nchunks; ++k) {
                if (k >= nstages && !mbar_wait(smem_u32(&ring->empty[s]), par ^ 1u)) {
                    report_timeout(EXB_STATUS_EMPTY_WAIT);
                    ring->aborted = 1;
                    break;
                }
                const uint32_t bar = smem_u32(&ring->full[s]);
                mbar_arrive_expect_tx(bar, (uint32_t)(NTT_STAGE * sizeof(float)));
                float *dst = stages + (size_t)s * NTT_STAGE;
                // boxes (or parts) outside the tensor are filled with zeros and still count as bytes
#pragma unroll
                for (int w = 0; w < NTT_WARPS; ++w)
                    tma_load_3d(smem_u32(dst + w * 32 * NTT_BOX_T), &maps.in, k * NTT_BOX_T - a, cls, r0 + w * 32, bar);
                if (++s == nstages) { s = 0; par ^= 1u; }
            }
            ring->issued = k;
        }
    } else {
        const int64_t row = (int64_t)r0 + warp * 32 + lane;            // inside the class
        const int64_t n = cls + (row << lp);
        const bool valid = n < N;
        const int64_t nn = valid ? n : 0;
        const int64_t b = nn / A.M, m = nn - b * A.M;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        const Neuron q = A.np.load(b, m, cfg);
        float v = A.v_init ? __ldg(A.v_init + nn) : 0.0f;
        float af = 0.0f;
        SpikeTotal cnt;
        cnt.c32 = 0u; cnt.c64 = 0ull;
        const int row_off = lane * NTT_BOX_T;          // this thread's row inside its warp's quarter of a stage
        const int sw = lane & 7;
        float *my_spk = spk + warp * 32 * NTT_BOX_T;
        bool ok = true;
        RingPos pos = {0, 0u};
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            float *st = stages + (size_t)pos.s * NTT_STAGE + warp * 32 * NTT_BOX_T;
            const int tb = k * NTT_BOX_T - a;          // time step of column 0 (the same for the whole CTA)
            float *tx = st + row_off;
            float *ts = my_spk + row_off;
            const bool head = tb < 0;
            if (head) {
                // First chunk of a class whose rows start inside a line: the granules before the row's start are
                // fill (a is a multiple of 4: a granule is inside the row or outside).
#pragma unroll 1
                for (int g = a >> 2; g < 8; ++g) {
                    const int o = (g ^ sw) << 2;
                    const float4 x4 = *reinterpret_cast<const float4 *>(tx + o);
                    float x[4] = {x4.x, x4.y, x4.z, x4.w};
                    float s4[4], u4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        lif_step<RESET>(v, af, x[e], q, cfg, cnt);
                        s4[e] = af;
                        u4[e] = v;
                    }
                    *reinterpret_cast<float4 *>(ts + o) = make_float4(s4[0], s4[1], s4[2], s4[3]);
                    *reinterpret_cast<float4 *>(tx + o) = make_float4(u4[0], u4[1], u4[2], u4[3]);
                }
            } else if (tb + NTT_BOX_T <= T) {
                ntt_chunk<RESET, false>(tx, ts, sw, tb, T, v, af, q, cfg, cnt);
            } else {
                ntt_chunk<RESET, true>(tx, ts, sw, tb, T, v, af, q, cfg, cnt);
            }
            if (head) {
                // A TMA store may not start at a negative coordinate: the warp stores the granules of this chunk
                // itself, a quarter-warp per row (lane -> row it*4 + lane/8, granule lane%8).
                __syncwarp();
                const int g = lane & 7, q4 = lane >> 3;
                if (g >= (a >> 2)) {
#pragma unroll 1
                    for (int it = 0; it < 8; ++it) {
                        const int r = it * 4 + q4;
                        const int64_t rn = (int64_t)r0 + warp * 32 + r;
                        const int64_t gn = cls + (rn << lp);
                        if (gn < N) {
                            const int o = r * NTT_BOX_T + ((g ^ (r & 7)) << 2);
                            const int64_t go = gn * T + tb + 4 * g;
                            __stcs(reinterpret_cast<float4 *>(A.spikes + go), *reinterpret_cast<const float4 *>(my_spk + o));
                            __stcs(reinterpret_cast<float4 *>(A.v_mem + go), *reinterpret_cast<const float4 *>(st + o));
                        }
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ring->empty[pos.s]));
            } else {
                fence_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const int x = k * NTT_BOX_T - a;
                    if (x < T) {      // beyond the end of the rows: nothing to store
                        tma_store_3d(&maps.spikes, x, cls, r0 + warp * 32, smem_u32(my_spk));
                        tma_store_3d(&maps.v_mem, x, cls, r0 + warp * 32, smem_u32(st));
                    }
                    tma_store_commit();
                    tma_store_wait_read();      // the stage and the spike tile may be overwritten from here on
                    mbar_arrive(smem_u32(&ring->empty[pos.s]));
                }
                __syncwarp();
            }
            pos.advance(nstages);
        }
        if (lane == 0) tma_store_wait_all();
        if (valid && A.v_post_last) A.v_post_last[n] = ok ? post_reset<RESET>(v, af, q) : NAN;
        if (A.spike_count) {
            const unsigned long long tot = warp_sum_u64((valid && ok) ? cnt.total(cfg) : 0ull);
            if (lane == 0 && tot) atomicAdd(A.spike_count, tot);
        }
    }
    ring_finish(ring, nstages);
}

cudaError_t launch_lif_forward_nt_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    static const bool off = env_int("EXB_DISABLE_NT_TMA", 0) == 1;
    if (off || a.v_post || a.spikes_u8) return cudaSuccess;
    const int64_t N = a.B * a.M;
    const int lp = nt_class_log2(a.T);
    if (lp < 0) return cudaSuccess;
    // the three tensors must agree on where a row starts inside its line
    const uintptr_t pos = reinterpret_cast<uintptr_t>(a.input) & 127u;
    if ((reinterpret_cast<uintptr_t>(a.spikes) & 127u) != pos || (reinterpret_cast<uintptr_t>(a.v_mem) & 127u) != pos)
        return cudaSuccess;
    NttMaps maps;
    if (!make_nt_tensor_map(&maps.in, a.input, N, a.T, lp) || !make_nt_tensor_map(&maps.spikes, a.spikes, N, a.T, lp) ||
        !make_nt_tensor_map(&maps.v_mem, a.v_mem, N, a.T, lp))
        return cudaSuccess;
    // one class per CTA: p classes x blocks of 128 rows of a class (the class index varies fastest)
    const int64_t ctas = (((N >> lp) + NTT_ROWS - 1) / NTT_ROWS) << lp;
    if (ctas > 0x7fffffffll) return cudaSuccess;
    static const int env_st = env_int("EXB_NT_TMA_STAGES", 0);
    const int nstages = (env_st >= 2 && env_st <= 6) ? env_st : 4;
    const size_t smem = (size_t)(nstages + 1) * NTT_STAGE * sizeof(float) + sizeof(Ring) + 1024 + 128;
    auto kern = reset_mode == EXB_RESET_SUBTRACT ? lif_fwd_nt_tma_kernel<EXB_RESET_SUBTRACT>
                                                 : lif_fwd_nt_tma_kernel<EXB_RESET_TO_VALUE>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)ctas, (NTT_WARPS + 1) * 32, smem, s>>>(maps, a, nstages, lp, (int)(pos >> 2));
    *used = true;
    return cudaPeekAtLastError();
}

}  // namespace exb
