// Pieces shared by the translation units that hold TMA-staged kernels: tile geometry, the
// producer loop, ring bookkeeping, and the host-side helpers (tensor maps, pipeline shape).
// Everything is `static`/inline so that every including translation unit is self-contained.
#pragma once

#include "exb_kernels.cuh"
#include "exb_tma.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>

namespace exb {

template <int NW, int V>
struct TileGeom {
    static constexpr int W = NW * 32 * V;
    static constexpr int BW = (W > 256) ? 256 : W;
    static constexpr int NBOX = W / BW;
};

// Resident CTAs per SM the kernels are compiled for (caps registers at 64 per thread).
// Light kernels fit 64 registers; the backward with alpha/scale gradients or an exponential
// surrogate keeps four neurons' constants and accumulators live and gets 96.
template <int NW, int V, bool HEAVY = false>
struct MinBlocks {
    static constexpr int value = (V == 4) ? (HEAVY ? 4 : 6) : (HEAVY ? 6 : 8);
};

// Shared-memory float offset of neuron column c inside one tensor's part of a stage, at time
// step 0 of the stage; consecutive time steps are BW floats apart.
template <int NW, int V>
__device__ __forceinline__ int tile_col_off(int tc, int c)
{
    using G = TileGeom<NW, V>;
    return (c / G::BW) * tc * G::BW + (c % G::BW);
}

// Pipeline shape chosen by the launcher: time steps per stage and number of stages.
struct PipeCfg {
    int tc;
    int stages;
};

// Producer: issues chunk k (k-th in processing order; `reverse` walks time backwards) of
// `nmaps` tensors into stage k % S.
template <int NW, int V>
__device__ __forceinline__ void produce(Ring *ring, float *stages, const CUtensorMap *const *maps, int nmaps,
                                        int nchunks, int m0, int b, PipeCfg pc, bool reverse)
{
    using G = TileGeom<NW, V>;
    const int tensor_floats = pc.tc * G::W;
    const int stage_floats = nmaps * tensor_floats;
    const int S = pc.stages;
    int k = 0;
    int s = 0;
    uint32_t par = 0u;             // (k / S) & 1, kept incrementally
    for (; k < nchunks; ++k) {
        if (k >= S && !mbar_wait(smem_u32(&ring->empty[s]), par ^ 1u)) {
            report_timeout(EXB_STATUS_EMPTY_WAIT);
            ring->aborted = 1;
            break;
        }
        const uint32_t bar = smem_u32(&ring->full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)(stage_floats * sizeof(float)));
        float *dst = stages + (size_t)s * stage_floats;
        const int chunk = reverse ? (nchunks - 1 - k) : k;
        for (int i = 0; i < nmaps; ++i) {
#pragma unroll
            for (int j = 0; j < G::NBOX; ++j)
                tma_load_3d(smem_u32(dst + i * tensor_floats + j * pc.tc * G::BW), maps[i], m0 + j * G::BW,
                            chunk * pc.tc, b, bar);
        }
        if (++s == S) { s = 0; par ^= 1u; }
    }
    ring->issued = k;
}

struct TmaMaps {
    CUtensorMap m[5];
};

template <int NW, int V>
static size_t tma_smem_bytes(int nmaps, PipeCfg pc)
{
    return (size_t)pc.stages * nmaps * pc.tc * TileGeom<NW, V>::W * sizeof(float) + sizeof(Ring) + 128;
}

// Position in the ring: stage index and the parity of the phase being used there.  Advanced
// incrementally (a `%` by a run-time stage count would cost an integer division per chunk).
struct RingPos {
    int s;
    uint32_t phase;
    __device__ __forceinline__ void advance(int S)
    {
        if (++s == S) { s = 0; phase ^= 1u; }
    }
};

// Consumer-side wait for the chunk at `pos`; marks the ring aborted when the wait runs out.
__device__ __forceinline__ bool wait_chunk(Ring *ring, const RingPos &pos)
{
    if (mbar_wait(smem_u32(&ring->full[pos.s]), pos.phase)) return true;
    report_timeout(EXB_STATUS_FULL_WAIT);
    ring->aborted = 1;
    return false;
}

__device__ __forceinline__ void release_chunk(Ring *ring, const RingPos &pos, int lane)
{
    __syncwarp();
    if (lane == 0) mbar_arrive(smem_u32(&ring->empty[pos.s]));
}

// V floats of one consumer thread from a stage.
template <int V>
__device__ __forceinline__ void lds_vec(float (&d)[V], const float *p)
{
    if (V == 4) {
        const float4 t = *reinterpret_cast<const float4 *>(p);
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else if (V == 2) {
        const float2 t = *reinterpret_cast<const float2 *>(p);
        d[0] = t.x; d[1] = t.y;
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] = p[j];
    }
}

// The same to a stage (a consumer thread overwriting its own columns).
template <int V>
__device__ __forceinline__ void sts_vec(float *p, const float (&d)[V])
{
    if (V == 4) *reinterpret_cast<float4 *>(p) = make_float4(d[0], d[1], d[2], d[3]);
    else if (V == 2) *reinterpret_cast<float2 *>(p) = make_float2(d[0], d[1]);
    else {
#pragma unroll
        for (int j = 0; j < V; ++j) p[j] = d[j];
    }
}

// V floats of one consumer thread from global memory (read-only path); p is aligned to V floats.
template <int V>
__device__ __forceinline__ void ldg_vec(float (&d)[V], const float *p)
{
    if (V == 4) {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        d[0] = t.x; d[1] = t.y; d[2] = t.z; d[3] = t.w;
    } else if (V == 2) {
        const float2 t = __ldg(reinterpret_cast<const float2 *>(p));
        d[0] = t.x; d[1] = t.y;
    } else {
#pragma unroll
        for (int j = 0; j < V; ++j) d[j] = __ldg(p + j);
    }
}

// ===========================================================================
// host side
// ===========================================================================
static PFN_cuTensorMapEncodeTiled get_encode_fn()
{
    static PFN_cuTensorMapEncodeTiled fn = []() -> PFN_cuTensorMapEncodeTiled {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess ||
            qres != cudaDriverEntryPointSuccess)
            return nullptr;
        return reinterpret_cast<PFN_cuTensorMapEncodeTiled>(p);
    }();
    return fn;
}

static bool make_btm_tensor_map(CUtensorMap *map, const float *base, int64_t B, int64_t T, int64_t M, int box_m, int box_t)
{
    PFN_cuTensorMapEncodeTiled enc = get_encode_fn();
    if (!enc || !base) return false;
    if ((reinterpret_cast<uintptr_t>(base) & 15u) || (M % 4) || M <= 0 || T <= 0 || B <= 0) return false;
    if (M > (1ll << 31) || T > (1ll << 31) || B > (1ll << 31)) return false;
    if ((double)T * (double)M * 4.0 >= 1.0e12) return false;    // stride limit is 2^40 bytes
    cuuint64_t gdim[3] = {(cuuint64_t)M, (cuuint64_t)T, (cuuint64_t)B};
    cuuint64_t gstr[2] = {(cuuint64_t)M * 4u, (cuuint64_t)T * (cuuint64_t)M * 4u};
    cuuint32_t box[3] = {(cuuint32_t)box_m, (cuuint32_t)box_t, 1u};
    cuuint32_t estr[3] = {1u, 1u, 1u};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<float *>(base), gdim, gstr, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

// Tile shape choice: wide tiles (512 neurons, 4+1 warps) when they alone fill the GPU,
// narrow tiles (128 neurons, 4+1 warps, longer time chunks) otherwise.  Tiles narrower than
// 128 neurons were measured and are slower: their 128-byte rows reach about 4.9 TB/s where
// 512-byte rows reach 6.1 TB/s, which costs more than the extra CTAs gain.  A middle shape (256
// neurons, 2 per thread) was measured on the fused synapse kernels: 14 % fewer instructions in the
// backward but half the warps, and slower overall.  The pipeline shape
// (time steps per stage, stages) keeps one stage at about 8-16 KB (the wide spiking forward on large grids
// takes longer stages, see run_lif_fwd).  EXB_TMA_TC / EXB_TMA_STAGES in the environment override it for every
// kernel, EXB_LIF_FWD_TC / EXB_LIF_FWD_STAGES for the spiking forward alone (tuning aids).
static bool use_wide(int64_t B, int64_t M)
{
    const int64_t wide_tiles = B * ((M + 511) / 512);
    return wide_tiles >= 2 * 148;
}
constexpr int NWARPS = 4;   // consumer warps per CTA in all tile shapes

static int env_int(const char *name, int dflt)
{
    const char *v = getenv(name);
    return (v && *v) ? atoi(v) : dflt;
}

static int sm_count()
{
    static const int n = []() {
        int dev = 0, v = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0)
            return 148;
        return v;
    }();
    return n;
}

// w: neurons per tile (512 or 128); nmaps: tensors streamed per stage; ctas: grid size.
static PipeCfg pipe_cfg(int w, int nmaps, int64_t ctas)
{
    static const int env_tc = env_int("EXB_TMA_TC", 0);
    static const int env_st = env_int("EXB_TMA_STAGES", 0);
    PipeCfg pc;
    pc.stages = 4;
    // ~8 KB per stage for one streamed tensor, ~16 KB for several (the backward kernels): with two
    // tensors in 8 KB a wide stage holds only 2 time steps and the per-chunk work (barrier wait,
    // release, loop set-up) weighs on every step.  Measured: c2 backward 0.682 -> 0.657 ms, c3 step
    // 0.467 -> 0.445 ms.
    int target = (nmaps >= 2) ? 16 * 1024 : 8 * 1024;
    // A grid of a few CTAs per SM should be resident at once: a second, short wave costs more than
    // longer stages gain (c4: 1024 CTAs, 7 per SM; with 3 resident the step took 0.60 instead of 0.53 ms).
    const int64_t per_sm = (ctas + sm_count() - 1) / sm_count();
    if (per_sm >= 1 && per_sm <= 8) {
        const int budget = (224 * 1024) / (int)per_sm - 1280;      // shared memory of one CTA, ring bookkeeping off
        if (target > budget / pc.stages) target = budget / pc.stages;
    }
    int tc = target / (w * 4 * nmaps);
    if (tc < 2) tc = 2;
    if (tc > 32) tc = 32;
    pc.tc = tc;
    if (env_tc > 0) pc.tc = env_tc;
    if (env_st > 1 && env_st <= MAX_STAGES) pc.stages = env_st;
    if (pc.tc > 256) pc.tc = 256;
    return pc;
}

// Forward kernels (one tensor in, one or two out) on wide tiles and a grid of many waves: two stages of 32 time
// steps (128 KB, so one CTA per SM).  These kernels write at least as much as they read, and they are fastest when
// each SM has 64-128 KB of loads in flight and four to eight warps storing.  Measured on 8 x 500 x 262144, spiking
// forward alone: 2.055 ms with 4 steps x 4 stages (six CTAs per SM, 192 KB in flight), 2.03 with 8 x 4 (three
// CTAs), 1.99 with 24 x 2 (two CTAs, 192 KB), 1.937 with 32 x 2, 1.936 with 8 x 4 when padded to one CTA per SM,
// 2.117 with 4 x 4 padded to one CTA per SM (32 KB in flight: too little); 32 x 300 x 36992: 0.700 -> 0.669 ms.
// The backward kernels (two or more tensors in, more arithmetic per step) want the opposite: 1.9 -> 3.1 ms with
// one CTA per SM.  One CTA per SM needs many waves, or the last one leaves SMs idle.
static void long_stages_for_wide_forward(PipeCfg &pc, int v, int64_t ctas, int64_t T)
{
    if (v == 4 && ctas >= 8 * (int64_t)sm_count() && T >= 128) { pc.tc = 32; pc.stages = 2; }
}

template <typename K>
static cudaError_t set_smem(K kern, size_t bytes)
{
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

static bool eligible(int64_t B, int64_t T, int64_t M)
{
    return M % 4 == 0 && B * ((M + 127) / 128) <= 0x7fffffffll && T <= 0x7fffffffll;
}

}  // namespace exb
