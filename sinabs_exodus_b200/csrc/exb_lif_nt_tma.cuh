// [N,T] layout, TMA-staged forward spike scan.
//
// The [N,T] layout (the reference's: one row per neuron, time contiguous) asks each neuron's thread
// for consecutive time steps of its own row.  Here a CTA owns 128 rows and walks time in chunks of 32 (or
// 64) steps, moved by TMA as 2-D boxes of [32 time steps x 32 rows] with the 128-byte swizzle, which is
// exactly the bank-conflict-free tile the lanes want (granule g of row r at position g ^ (r & 7)).
// A producer warp streams the input boxes through a ring of stages (mbarriers, bounded waits); the four
// consumer warps -- lane = row -- run the recurrence over the 64 steps of a stage, overwrite the stage
// with the membrane potential and fill a spike tile beside it, and hand both to TMA stores (bulk async
// group), which clip at the tensor's edges.  A row need not start on any boundary: chunk boundaries are
// at fixed time steps, the hardware splits the boxes into sectors.
//
// Chunk boundaries are at fixed time steps for all rows, so this only pays when every row starts on a
// 128-byte line (T % 32 == 0 and 128-byte aligned tensors): then each box row is one whole line.  Measured
// on 1 183 744 rows: T = 320: 5.96 TB/s against 5.36 for the cp.async variant; T = 300 (rows start at any
// multiple of 16 bytes, every piece ends in partial sectors): 4.12 against 4.47 -- those shapes keep the
// cp.async variant, whose chunks follow each row's own lines.  Stages of 32 steps, four of them (80 KB per
// CTA, two CTAs per SM) measured best: 64 steps x 2 stages 5.81 TB/s, 32 x 6 (one CTA per SM) 3.75.
// Included by exb_tma_kernels.cu (shares its status word).
#pragma once

namespace exb {

constexpr int NTT_WARPS = 4;           // consumer warps per CTA
constexpr int NTT_ROWS = NTT_WARPS * 32;   // rows per CTA (lane = row)
constexpr int NTT_BOX_T = 32;          // time steps per box (128 bytes: the swizzle span)
constexpr int NTT_TILE = 32 * NTT_BOX_T;               // floats of one [32 rows x 32 steps] box
// TC: time steps per stage (32 or 64); a stage holds NTT_WARPS * TC/32 boxes (16 or 32 KB)
template <int TC>
struct NttGeom {
    static constexpr int BOXES_T = TC / NTT_BOX_T;
    static constexpr int STAGE = NTT_WARPS * BOXES_T * NTT_TILE;
};

struct NttMaps {
    CUtensorMap in, spikes, v_mem;
};

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap *map, int x, int y, uint32_t bar)
{
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tma_store_2d(const CUtensorMap *map, int x, int y, uint32_t src)
{
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%1, %2}], [%3];"
                 ::"l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(src)
                 : "memory");
}

__device__ __forceinline__ void tma_store_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
// all stores of this thread's groups have finished READING shared memory (the data may still be on its way to DRAM)
__device__ __forceinline__ void tma_store_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void tma_store_wait_all() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// makes this thread's shared-memory writes visible to the async (TMA) proxy
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

template <int RESET, int NTT_TC>
__global__ void __launch_bounds__((NTT_WARPS + 1) * 32, 2)
lif_fwd_nt_tma_kernel(const __grid_constant__ NttMaps maps, const LifFwdArgs A, const int nstages)
{
    constexpr int NTT_STAGE = NttGeom<NTT_TC>::STAGE;
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // the swizzle works on 1 KB atoms: every box must start on one
    float *stages = reinterpret_cast<float *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023u) & ~uintptr_t(1023));
    float *spk = stages + (size_t)nstages * NTT_STAGE;                 // one spike stage, a quarter per warp
    Ring *ring = reinterpret_cast<Ring *>(spk + NTT_STAGE);
    ring_init(ring, nstages, NTT_WARPS);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t N = A.B * A.M;
    const int T = (int)A.T;
    const int64_t n0 = (int64_t)blockIdx.x * NTT_ROWS;
    const int nchunks = (T + NTT_TC - 1) / NTT_TC;
    constexpr int BOXES_T = NttGeom<NTT_TC>::BOXES_T;

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
#pragma unroll
                for (int w = 0; w < NTT_WARPS; ++w)
#pragma unroll
                    for (int j = 0; j < BOXES_T; ++j)      // boxes beyond the tensor are filled with zeros and still count
                        tma_load_2d(smem_u32(dst + (w * BOXES_T + j) * NTT_TILE), &maps.in, k * NTT_TC + j * NTT_BOX_T,
                                    (int)(n0 + w * 32), bar);
                if (++s == nstages) { s = 0; par ^= 1u; }
            }
            ring->issued = k;
        }
    } else {
        const int64_t n = n0 + warp * 32 + lane;
        const bool valid = n < N;
        const int64_t nn = valid ? n : 0;
        const int64_t b = nn / A.M, m = nn - b * A.M;
        const SpikeCfg cfg = make_spike_cfg(A.maxs);
        const Neuron q = A.np.load(b, m, cfg);
        float v = A.v_init ? __ldg(A.v_init + nn) : 0.0f;
        float af = 0.0f;
        SpikeTotal cnt;
        cnt.c32 = 0u; cnt.c64 = 0ull;
        const int row_off = lane * NTT_BOX_T;          // this lane's row inside a box
        const int sw = lane & 7;
        float *my_spk = spk + warp * BOXES_T * NTT_TILE;
        bool ok = true;
        RingPos pos = {0, 0u};
        for (int k = 0; k < nchunks; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            float *st = stages + (size_t)pos.s * NTT_STAGE + warp * BOXES_T * NTT_TILE;
            const int t0 = k * NTT_TC;
            const bool full = t0 + NTT_TC <= T;
#pragma unroll
            for (int j = 0; j < BOXES_T; ++j) {
                float *tx = st + j * NTT_TILE + row_off;
                float *ts = my_spk + j * NTT_TILE + row_off;
                // the next granule is read before this one's results are written (no shared-memory round trip per granule)
                float4 xn = *reinterpret_cast<const float4 *>(tx + ((0 ^ sw) << 2));
#pragma unroll
                for (int g = 0; g < 8; ++g) {
                    const int o = (g ^ sw) << 2;
                    const float4 x4 = xn;
                    if (g < 7) xn = *reinterpret_cast<const float4 *>(tx + (((g + 1) ^ sw) << 2));
                    float x[4] = {x4.x, x4.y, x4.z, x4.w};
                    float s4[4], u4[4];
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        if (full || t0 + j * NTT_BOX_T + 4 * g + e < T) lif_step<RESET>(v, af, x[e], q, cfg, cnt);
                        s4[e] = af;
                        u4[e] = v;
                    }
                    *reinterpret_cast<float4 *>(ts + o) = make_float4(s4[0], s4[1], s4[2], s4[3]);
                    *reinterpret_cast<float4 *>(tx + o) = make_float4(u4[0], u4[1], u4[2], u4[3]);
                }
            }
            fence_async_smem();
            __syncwarp();
            if (lane == 0) {
#pragma unroll
                for (int j = 0; j < BOXES_T; ++j) {
                    const int x = t0 + j * NTT_BOX_T;
                    if (x < T) {      // a box that starts beyond the end of time has nothing to store
                        tma_store_2d(&maps.spikes, x, (int)(n0 + warp * 32), smem_u32(my_spk + j * NTT_TILE));
                        tma_store_2d(&maps.v_mem, x, (int)(n0 + warp * 32), smem_u32(st + j * NTT_TILE));
                    }
                }
                tma_store_commit();
                tma_store_wait_read();      // the stage and the spike tile may be overwritten from here on
                mbar_arrive(smem_u32(&ring->empty[pos.s]));
            }
            __syncwarp();
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

// 2-D map of an [N,T] tensor: x = time (contiguous), y = row; boxes of [32 x 32] with the 128-byte swizzle.
static bool make_nt_tensor_map(CUtensorMap *map, const float *base, int64_t N, int64_t T)
{
    PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
    if (!enc || !base) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 127u) || (T % 32) || T < 64 || N <= 0) return false;
    if (T > (1ll << 31) - 64 || N > (1ll << 31) - NTT_ROWS) return false;
    cuuint64_t gdim[2] = {(cuuint64_t)T, (cuuint64_t)N};
    cuuint64_t gstr[1] = {(cuuint64_t)T * 4u};
    cuuint32_t box[2] = {(cuuint32_t)NTT_BOX_T, 32u};
    cuuint32_t estr[2] = {1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<float *>(base), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

cudaError_t launch_lif_forward_nt_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    static const bool off = env_int("EXB_DISABLE_NT_TMA", 0) == 1;
    if (off || a.v_post || a.spikes_u8) return cudaSuccess;
    const int64_t N = a.B * a.M;
    NttMaps maps;
    if (!make_nt_tensor_map(&maps.in, a.input, N, a.T) || !make_nt_tensor_map(&maps.spikes, a.spikes, N, a.T) ||
        !make_nt_tensor_map(&maps.v_mem, a.v_mem, N, a.T))
        return cudaSuccess;
    const int64_t ctas = (N + NTT_ROWS - 1) / NTT_ROWS;
    if (ctas > 0x7fffffffll) return cudaSuccess;
    static const int env_st = env_int("EXB_NT_TMA_STAGES", 0);
    static const int env_tc = env_int("EXB_NT_TMA_TC", 0);
    const int tc = (env_tc == 64) ? 64 : 32;
    const int nstages = (env_st >= 2 && env_st <= 6) ? env_st : (tc == 32 ? 4 : 2);
    const size_t stage_bytes = (size_t)(tc == 32 ? NttGeom<32>::STAGE : NttGeom<64>::STAGE) * sizeof(float);
    const size_t smem = (size_t)(nstages + 1) * stage_bytes + sizeof(Ring) + 1024 + 128;
    const bool sub = reset_mode == EXB_RESET_SUBTRACT;
    auto kern = tc == 32 ? (sub ? lif_fwd_nt_tma_kernel<EXB_RESET_SUBTRACT, 32> : lif_fwd_nt_tma_kernel<EXB_RESET_TO_VALUE, 32>)
                         : (sub ? lif_fwd_nt_tma_kernel<EXB_RESET_SUBTRACT, 64> : lif_fwd_nt_tma_kernel<EXB_RESET_TO_VALUE, 64>);
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)ctas, (NTT_WARPS + 1) * 32, smem, s>>>(maps, a, nstages);
    *used = true;
    return cudaPeekAtLastError();
}

}  // namespace exb
