// TMA-staged time-major kernels (spike scan forward, fused EXODUS backward,
// leaky integrator forward and backward).  See exb_tma.cuh for the pipeline.
//
// Tile geometry: NW consumer warps, every consumer thread owns 4 adjacent
// neurons, so a CTA covers W = NW*128 neurons of one batch item.  One stage
// holds TC time steps of every streamed tensor; a tensor's part of the stage
// is W/BW boxes of [TC][BW] floats (a TMA box is at most 256 elements wide).
#include "exb_kernels.cuh"
#include "exb_tma.cuh"

#include <cudaTypedefs.h>
#include <cstdlib>

namespace exb {

template <int NW>
struct TileGeom {
    static constexpr int W = NW * 128;
    static constexpr int BW = (W > 256) ? 256 : W;
    static constexpr int NBOX = W / BW;
};

// Shared-memory float offset of (time step tt, neuron column c) inside one tensor's part of a stage.
template <int NW, int TC>
__device__ __forceinline__ int tile_off(int tt, int c)
{
    using G = TileGeom<NW>;
    return ((c / G::BW) * TC + tt) * G::BW + (c % G::BW);
}

// Producer: issues chunk k of `nmaps` tensors into stage k % S.
template <int NW, int TC, int S>
__device__ __forceinline__ void produce(Ring<S> *ring, float *stages, const CUtensorMap *const *maps, int nmaps,
                                        int nchunks, int m0, int b)
{
    using G = TileGeom<NW>;
    constexpr int TENSOR_FLOATS = TC * G::W;
    const int stage_floats = nmaps * TENSOR_FLOATS;
    int k = 0;
    for (; k < nchunks; ++k) {
        const int s = k % S;
        if (k >= S && !mbar_wait(smem_u32(&ring->empty[s]), (uint32_t)(((k / S) - 1) & 1))) {
            report_timeout(EXB_STATUS_EMPTY_WAIT);
            ring->aborted = 1;
            break;
        }
        const uint32_t bar = smem_u32(&ring->full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)(stage_floats * sizeof(float)));
        float *dst = stages + (size_t)s * stage_floats;
        for (int i = 0; i < nmaps; ++i) {
#pragma unroll
            for (int j = 0; j < G::NBOX; ++j)
                tma_load_3d(smem_u32(dst + i * TENSOR_FLOATS + j * TC * G::BW), maps[i], m0 + j * G::BW, k * TC, b, bar);
        }
    }
    ring->issued = k;
}

// Reverse-time producer: chunk index kk counts from the end of the sequence.
template <int NW, int TC, int S>
__device__ __forceinline__ void produce_reverse(Ring<S> *ring, float *stages, const CUtensorMap *const *maps, int nmaps,
                                                int nchunks, int m0, int b)
{
    using G = TileGeom<NW>;
    constexpr int TENSOR_FLOATS = TC * G::W;
    const int stage_floats = nmaps * TENSOR_FLOATS;
    int k = 0;
    for (; k < nchunks; ++k) {
        const int s = k % S;
        if (k >= S && !mbar_wait(smem_u32(&ring->empty[s]), (uint32_t)(((k / S) - 1) & 1))) {
            report_timeout(EXB_STATUS_EMPTY_WAIT);
            ring->aborted = 1;
            break;
        }
        const uint32_t bar = smem_u32(&ring->full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)(stage_floats * sizeof(float)));
        float *dst = stages + (size_t)s * stage_floats;
        const int chunk = nchunks - 1 - k;
        for (int i = 0; i < nmaps; ++i) {
#pragma unroll
            for (int j = 0; j < G::NBOX; ++j)
                tma_load_3d(smem_u32(dst + i * TENSOR_FLOATS + j * TC * G::BW), maps[i], m0 + j * G::BW, chunk * TC, b, bar);
        }
    }
    ring->issued = k;
}

struct TmaMaps {
    CUtensorMap m[5];
};

template <int NW, int TC, int S>
constexpr size_t tma_smem_bytes(int nmaps)
{
    return (size_t)S * nmaps * TC * TileGeom<NW>::W * sizeof(float) + sizeof(Ring<S>) + 128;
}

// ===========================================================================
// spike scan forward
// ===========================================================================
template <int RESET, int NW, int TC, int S>
__global__ void __launch_bounds__((NW + 1) * 32)
lif_fwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LifFwdArgs A, const int tiles_m)
{
    using G = TileGeom<NW>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    Ring<S> *ring = reinterpret_cast<Ring<S> *>(smem_raw + (size_t)S * TC * G::W * sizeof(float));
    ring_init<S>(ring, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[1] = {&maps.m[0]};
            produce<NW, TC, S>(ring, stages, mp, 1, nchunks, m0, b);
        }
    } else {
        const int c = threadIdx.x * 4;                 // column inside the tile
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;                    // M % 4 == 0: all four neurons or none
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        Neuron q[4];
        float v[4];
        unsigned a[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[j] = A.np.load(b, mm + j);
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
            a[j] = 0u;
        }
        const int64_t base = ((int64_t)b * T) * A.M + mm;
        float *sp = A.spikes + base;
        float *vm = A.v_mem + base;
        unsigned long long cnt = 0ull;
        bool ok = true;
        for (int k = 0; k < nchunks && ok; ++k) {
            const int s = k % S;
            if (!mbar_wait(smem_u32(&ring->full[s]), (uint32_t)((k / S) & 1))) {
                report_timeout(EXB_STATUS_FULL_WAIT);
                ring->aborted = 1;
                ok = false;
                break;
            }
            const float *st = stages + (size_t)s * TC * G::W;
            const int tmax = min(TC, T - k * TC);
#pragma unroll
            for (int tt = 0; tt < TC; ++tt) {
                if (tt < tmax) {
                    const float4 x = lds128(st + tile_off<NW, TC>(tt, c));
                    const float xs[4] = {x.x, x.y, x.z, x.w};
                    float sv[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        lif_step<RESET>(v[j], a[j], xs[j], q[j], A.maxs);
                        sv[j] = __uint2float_rn(a[j]);
                        cnt += a[j];
                    }
                    if (valid) {
                        const int64_t off = (int64_t)(k * TC + tt) * A.M;
                        stv<4>(sp + off, sv);
                        stv<4>(vm + off, v);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ring->empty[s]));
        }
        if (ok && valid && A.v_post_last) {
#pragma unroll
            for (int j = 0; j < 4; ++j) A.v_post_last[n + j] = post_reset<RESET>(v[j], a[j], q[j]);
        }
        if (A.spike_count) {
            cnt = warp_sum_u64((valid && ok) ? cnt : 0ull);
            if (lane == 0 && cnt) atomicAdd(A.spike_count, cnt);
        }
    }
    ring_finish<S>(ring);
}

// ===========================================================================
// fused reverse-time backward
// ===========================================================================
template <int SURR, int RESET, bool WA, bool WS, int NW, int TC, int S>
__global__ void __launch_bounds__((NW + 1) * 32)
lif_bwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LifBwdArgs A, const int tiles_m, const int nmaps)
{
    using G = TileGeom<NW>;
    constexpr int TENSOR_FLOATS = TC * G::W;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    Ring<S> *ring = reinterpret_cast<Ring<S> *>(smem_raw + (size_t)S * nmaps * TENSOR_FLOATS * sizeof(float));
    ring_init<S>(ring, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;
    // stage layout: [go][v_mem]([grad_v_mem])([surr])([input])
    const bool has_gv = A.gv != nullptr;
    const int i_gv = 2;
    const int i_sl = 2 + (has_gv ? 1 : 0);
    const int i_x = i_sl + ((SURR == EXB_SURR_GENERIC) ? 1 : 0);

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[5] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4]};
            produce_reverse<NW, TC, S>(ring, stages, mp, nmaps, nchunks, m0, b);
        }
    } else {
        const int c = threadIdx.x * 4;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        Neuron q[4];
        SurrConst sc[4];
        float cp[4], Rprev[4], f0[4], glast[4];
        bool n0[4];
        BwdState st[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            q[j] = A.np.load(b, mm + j);
            sc[j] = surr_prepare<SURR>(q[j], A.p0, A.p1);
            cp[j] = __fmul_rn(q[j].alpha, q[j].c);
            st[j].R = 0.0f; st[j].ag = 0.0f; st[j].sg = 0.0f;
            Rprev[j] = 0.0f; f0[j] = 0.0f; n0[j] = true;
            glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
        }
        float *gi = A.grad_input + ((int64_t)b * T) * A.M + mm;
        bool ok = true;
        for (int k = 0; k < nchunks && ok; ++k) {
            const int s = k % S;
            if (!mbar_wait(smem_u32(&ring->full[s]), (uint32_t)((k / S) & 1))) {
                report_timeout(EXB_STATUS_FULL_WAIT);
                ring->aborted = 1;
                ok = false;
                break;
            }
            const float *stg = stages + (size_t)s * nmaps * TENSOR_FLOATS;
            const int chunk = nchunks - 1 - k;
            const int tmax = min(TC, T - chunk * TC);
#pragma unroll
            for (int tt = TC - 1; tt >= 0; --tt) {
                if (tt < tmax) {
                    const int o = tile_off<NW, TC>(tt, c);
                    const float4 g4 = lds128(stg + o);
                    const float4 v4 = lds128(stg + TENSOR_FLOATS + o);
                    float go[4] = {g4.x, g4.y, g4.z, g4.w};
                    const float vv[4] = {v4.x, v4.y, v4.z, v4.w};
                    float gv[4] = {0.0f, 0.0f, 0.0f, 0.0f}, sl[4] = {0.0f, 0.0f, 0.0f, 0.0f}, xx[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (has_gv) {
                        const float4 t4 = lds128(stg + i_gv * TENSOR_FLOATS + o);
                        gv[0] = t4.x; gv[1] = t4.y; gv[2] = t4.z; gv[3] = t4.w;
                    }
                    if (SURR == EXB_SURR_GENERIC) {
                        const float4 t4 = lds128(stg + i_sl * TENSOR_FLOATS + o);
                        sl[0] = t4.x; sl[1] = t4.y; sl[2] = t4.z; sl[3] = t4.w;
                    }
                    if (WS) {
                        const float4 t4 = lds128(stg + i_x * TENSOR_FLOATS + o);
                        xx[0] = t4.x; xx[1] = t4.y; xx[2] = t4.z; xx[3] = t4.w;
                    }
                    const int t = chunk * TC + tt;
                    if (A.g_last && t == T - 1) {
#pragma unroll
                        for (int j = 0; j < 4; ++j) fold_last_state_grad<RESET>(go[j], gv[j], glast[j], vv[j], q[j], A.maxs);
                    }
                    float r[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        Rprev[j] = st[j].R;
                        const float Rt = lif_bwd_step<SURR, RESET, WA, WS>(st[j], vv[j], go[j], gv[j], sl[j], xx[j], q[j],
                                                                          sc[j], cp[j], A.maxs, f0[j], n0[j]);
                        r[j] = __fmul_rn(q[j].scale, Rt);
                    }
                    if (valid) stv<4>(gi + (int64_t)t * A.M, r);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ring->empty[s]));
        }
        if (ok && valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (A.grad_init) A.grad_init[n + j] = __fmul_rn(q[j].alpha, st[j].R);
                if (WA) {
                    const float vi = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
                    A.grad_alpha[n + j] = alpha_grad_finish<RESET>(st[j], vi, Rprev[j], f0[j], n0[j]);
                }
                if (WS) A.grad_scale[n + j] = st[j].sg;
            }
        }
    }
    ring_finish<S>(ring);
}

// ===========================================================================
// leaky integrator
// ===========================================================================
template <int NW, int TC, int S>
__global__ void __launch_bounds__((NW + 1) * 32)
leaky_fwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LeakyFwdArgs A, const int tiles_m)
{
    using G = TileGeom<NW>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    Ring<S> *ring = reinterpret_cast<Ring<S> *>(smem_raw + (size_t)S * TC * G::W * sizeof(float));
    ring_init<S>(ring, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[1] = {&maps.m[0]};
            produce<NW, TC, S>(ring, stages, mp, 1, nchunks, m0, b);
        }
    } else {
        const int c = threadIdx.x * 4;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        float al[4], sc[4], v[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            al[j] = A.alpha.get(b, mm + j, 1.0f);
            sc[j] = A.scale.get(b, mm + j, 1.0f);
            v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
        }
        float *out = A.out + ((int64_t)b * T) * A.M + mm;
        bool ok = true;
        for (int k = 0; k < nchunks && ok; ++k) {
            const int s = k % S;
            if (!mbar_wait(smem_u32(&ring->full[s]), (uint32_t)((k / S) & 1))) {
                report_timeout(EXB_STATUS_FULL_WAIT);
                ring->aborted = 1;
                ok = false;
                break;
            }
            const float *st = stages + (size_t)s * TC * G::W;
            const int tmax = min(TC, T - k * TC);
#pragma unroll
            for (int tt = 0; tt < TC; ++tt) {
                if (tt < tmax) {
                    const float4 x = lds128(st + tile_off<NW, TC>(tt, c));
                    const float xs[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) v[j] = __fmaf_rn(v[j], al[j], __fmul_rn(sc[j], xs[j]));
                    if (valid) stv<4>(out + (int64_t)(k * TC + tt) * A.M, v);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ring->empty[s]));
        }
        if (ok && valid && A.v_last) {
#pragma unroll
            for (int j = 0; j < 4; ++j) A.v_last[n + j] = v[j];
        }
    }
    ring_finish<S>(ring);
}

template <bool WA, bool WS, int NW, int TC, int S>
__global__ void __launch_bounds__((NW + 1) * 32)
leaky_bwd_tma_kernel(const __grid_constant__ TmaMaps maps, const LeakyBwdArgs A, const int tiles_m, const int nmaps)
{
    using G = TileGeom<NW>;
    constexpr int TENSOR_FLOATS = TC * G::W;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    Ring<S> *ring = reinterpret_cast<Ring<S> *>(smem_raw + (size_t)S * nmaps * TENSOR_FLOATS * sizeof(float));
    ring_init<S>(ring, NW);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b = blockIdx.x / tiles_m;
    const int m0 = (blockIdx.x - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int nchunks = (T + TC - 1) / TC;
    // stage layout: [grad_out]([out])([input])
    const int i_x = WA ? 2 : 1;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[5] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4]};
            produce_reverse<NW, TC, S>(ring, stages, mp, nmaps, nchunks, m0, b);
        }
    } else {
        const int c = threadIdx.x * 4;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        float al[4], sc[4], G_[4], ag[4], sg[4], glast[4];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            al[j] = A.alpha.get(b, mm + j, 1.0f);
            sc[j] = A.scale.get(b, mm + j, 1.0f);
            G_[j] = 0.0f; ag[j] = 0.0f; sg[j] = 0.0f;
            glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
        }
        float *gi = A.grad_input + ((int64_t)b * T) * A.M + mm;
        bool ok = true;
        for (int k = 0; k < nchunks && ok; ++k) {
            const int s = k % S;
            if (!mbar_wait(smem_u32(&ring->full[s]), (uint32_t)((k / S) & 1))) {
                report_timeout(EXB_STATUS_FULL_WAIT);
                ring->aborted = 1;
                ok = false;
                break;
            }
            const float *stg = stages + (size_t)s * nmaps * TENSOR_FLOATS;
            const int chunk = nchunks - 1 - k;
            const int tmax = min(TC, T - chunk * TC);
#pragma unroll
            for (int tt = TC - 1; tt >= 0; --tt) {
                if (tt < tmax) {
                    const int o = tile_off<NW, TC>(tt, c);
                    const float4 g4 = lds128(stg + o);
                    float go[4] = {g4.x, g4.y, g4.z, g4.w};
                    float vo[4] = {0.0f, 0.0f, 0.0f, 0.0f}, xx[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (WA) {
                        const float4 t4 = lds128(stg + TENSOR_FLOATS + o);
                        vo[0] = t4.x; vo[1] = t4.y; vo[2] = t4.z; vo[3] = t4.w;
                    }
                    if (WS) {
                        const float4 t4 = lds128(stg + i_x * TENSOR_FLOATS + o);
                        xx[0] = t4.x; xx[1] = t4.y; xx[2] = t4.z; xx[3] = t4.w;
                    }
                    const int t = chunk * TC + tt;
                    float r[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        if (t == T - 1) go[j] = __fadd_rn(go[j], glast[j]);
                        if (WA) ag[j] = __fmaf_rn(G_[j], vo[j], ag[j]);
                        G_[j] = __fmaf_rn(G_[j], al[j], go[j]);
                        if (WS) sg[j] = __fmaf_rn(G_[j], xx[j], sg[j]);
                        r[j] = __fmul_rn(sc[j], G_[j]);
                    }
                    if (valid) stv<4>(gi + (int64_t)t * A.M, r);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&ring->empty[s]));
        }
        if (ok && valid) {
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                if (A.grad_init) A.grad_init[n + j] = __fmul_rn(al[j], G_[j]);
                if (WA) A.grad_alpha[n + j] = __fmaf_rn(G_[j], A.v_init ? __ldg(A.v_init + n + j) : 0.0f, ag[j]);
                if (WS) A.grad_scale[n + j] = sg[j];
            }
        }
    }
    ring_finish<S>(ring);
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

bool make_btm_tensor_map(CUtensorMap *map, const float *base, int64_t B, int64_t T, int64_t M, int box_m, int box_t)
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

// Tile shape choice: wide tiles (512 neurons, 4+1 warps) when they alone fill the
// GPU, narrow tiles (128 neurons, 1+1 warps, longer time chunks) otherwise.
static bool use_wide(int64_t B, int64_t M)
{
    const int64_t wide_tiles = B * ((M + 511) / 512);
    return wide_tiles >= 2 * 148;
}

template <typename K>
static cudaError_t set_smem(K kern, size_t bytes)
{
    if (bytes <= 48 * 1024) return cudaSuccess;
    return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
}

template <int RESET, int NW, int TC, int S>
static cudaError_t run_lif_fwd(const LifFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW>;
    TmaMaps maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, TC, S>(1);
    auto kern = lif_fwd_tma_kernel<RESET, NW, TC, S>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m);
    *used = true;
    return cudaPeekAtLastError();
}

cudaError_t launch_lif_forward_tma(const LifFwdArgs &a, int reset_mode, cudaStream_t s, bool *used)
{
    *used = false;
    if (a.M % 4 || !aligned16(a.spikes) || !aligned16(a.v_mem) || !aligned16(a.input)) return cudaSuccess;
    if (a.B * ((a.M + 127) / 128) > 0x7fffffffll || a.T > 0x7fffffffll) return cudaSuccess;
    const bool wide = use_wide(a.B, a.M);
    if (reset_mode == EXB_RESET_SUBTRACT)
        return wide ? run_lif_fwd<EXB_RESET_SUBTRACT, 4, 8, 4>(a, s, used) : run_lif_fwd<EXB_RESET_SUBTRACT, 1, 32, 4>(a, s, used);
    return wide ? run_lif_fwd<EXB_RESET_TO_VALUE, 4, 8, 4>(a, s, used) : run_lif_fwd<EXB_RESET_TO_VALUE, 1, 32, 4>(a, s, used);
}

template <int SURR, int RESET, bool WA, bool WS, int NW, int TC, int S>
static cudaError_t run_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW>;
    TmaMaps maps;
    const float *ptrs[5] = {a.go, a.v_mem, nullptr, nullptr, nullptr};
    int nmaps = 2;
    if (a.gv) ptrs[nmaps++] = a.gv;
    if (SURR == EXB_SURR_GENERIC) ptrs[nmaps++] = a.surr;
    if (WS) ptrs[nmaps++] = a.input;
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    for (int i = nmaps; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, TC, S>(nmaps);
    if (smem > 200 * 1024) return cudaSuccess;
    auto kern = lif_bwd_tma_kernel<SURR, RESET, WA, WS, NW, TC, S>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps);
    *used = true;
    return cudaPeekAtLastError();
}

template <int SURR, int RESET, bool WA, bool WS>
static cudaError_t pick_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    return use_wide(a.B, a.M) ? run_lif_bwd<SURR, RESET, WA, WS, 4, 4, 4>(a, s, used)
                              : run_lif_bwd<SURR, RESET, WA, WS, 1, 16, 4>(a, s, used);
}

template <int SURR, int RESET>
static cudaError_t flags_lif_bwd(const LifBwdArgs &a, cudaStream_t s, bool *used)
{
    const bool wa = a.grad_alpha != nullptr, ws = a.grad_scale != nullptr;
    if (wa && ws) return pick_lif_bwd<SURR, RESET, true, true>(a, s, used);
    if (wa) return pick_lif_bwd<SURR, RESET, true, false>(a, s, used);
    if (ws) return pick_lif_bwd<SURR, RESET, false, true>(a, s, used);
    return pick_lif_bwd<SURR, RESET, false, false>(a, s, used);
}

template <int RESET>
static cudaError_t surr_lif_bwd(const LifBwdArgs &a, int kind, cudaStream_t s, bool *used)
{
    switch (kind) {
    case EXB_SURR_GENERIC: return flags_lif_bwd<EXB_SURR_GENERIC, RESET>(a, s, used);
    case EXB_SURR_SINGLE_EXPONENTIAL: return flags_lif_bwd<EXB_SURR_SINGLE_EXPONENTIAL, RESET>(a, s, used);
    case EXB_SURR_HEAVISIDE: return flags_lif_bwd<EXB_SURR_HEAVISIDE, RESET>(a, s, used);
    default: return flags_lif_bwd<EXB_SURR_PERIODIC_EXPONENTIAL, RESET>(a, s, used);
    }
}

cudaError_t launch_lif_backward_tma(const LifBwdArgs &a, int reset_mode, int surr_kind, cudaStream_t s, bool *used)
{
    *used = false;
    if (a.M % 4 || !aligned16(a.grad_input)) return cudaSuccess;
    if (a.B * ((a.M + 127) / 128) > 0x7fffffffll || a.T > 0x7fffffffll) return cudaSuccess;
    return reset_mode == EXB_RESET_SUBTRACT ? surr_lif_bwd<EXB_RESET_SUBTRACT>(a, surr_kind, s, used)
                                            : surr_lif_bwd<EXB_RESET_TO_VALUE>(a, surr_kind, s, used);
}

template <int NW, int TC, int S>
static cudaError_t run_leaky_fwd(const LeakyFwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW>;
    TmaMaps maps;
    if (!make_btm_tensor_map(&maps.m[0], a.input, a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, TC, S>(1);
    auto kern = leaky_fwd_tma_kernel<NW, TC, S>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m);
    *used = true;
    return cudaPeekAtLastError();
}

cudaError_t launch_leaky_forward_tma(const LeakyFwdArgs &a, cudaStream_t s, bool *used)
{
    *used = false;
    if (a.M % 4 || !aligned16(a.out) || !aligned16(a.input)) return cudaSuccess;
    if (a.B * ((a.M + 127) / 128) > 0x7fffffffll || a.T > 0x7fffffffll) return cudaSuccess;
    return use_wide(a.B, a.M) ? run_leaky_fwd<4, 8, 4>(a, s, used) : run_leaky_fwd<1, 32, 4>(a, s, used);
}

template <bool WA, bool WS, int NW, int TC, int S>
static cudaError_t run_leaky_bwd(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    using G = TileGeom<NW>;
    TmaMaps maps;
    const float *ptrs[5] = {a.go, nullptr, nullptr, nullptr, nullptr};
    int nmaps = 1;
    if (WA) ptrs[nmaps++] = a.out;
    if (WS) ptrs[nmaps++] = a.input;
    for (int i = 0; i < nmaps; ++i)
        if (!make_btm_tensor_map(&maps.m[i], ptrs[i], a.B, a.T, a.M, G::BW, TC)) return cudaSuccess;
    for (int i = nmaps; i < 5; ++i) maps.m[i] = maps.m[0];
    const int tiles_m = (int)((a.M + G::W - 1) / G::W);
    const size_t smem = tma_smem_bytes<NW, TC, S>(nmaps);
    auto kern = leaky_bwd_tma_kernel<WA, WS, NW, TC, S>;
    cudaError_t e = set_smem(kern, smem);
    if (e != cudaSuccess) return e;
    kern<<<(unsigned)(a.B * tiles_m), (NW + 1) * 32, smem, s>>>(maps, a, tiles_m, nmaps);
    *used = true;
    return cudaPeekAtLastError();
}

template <bool WA, bool WS>
static cudaError_t pick_leaky_bwd(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    return use_wide(a.B, a.M) ? run_leaky_bwd<WA, WS, 4, 4, 4>(a, s, used) : run_leaky_bwd<WA, WS, 1, 16, 4>(a, s, used);
}

cudaError_t launch_leaky_backward_tma(const LeakyBwdArgs &a, cudaStream_t s, bool *used)
{
    *used = false;
    if (a.M % 4 || !aligned16(a.grad_input)) return cudaSuccess;
    if (a.B * ((a.M + 127) / 128) > 0x7fffffffll || a.T > 0x7fffffffll) return cudaSuccess;
    const bool wa = a.grad_alpha != nullptr, ws = a.grad_scale != nullptr;
    if (wa && ws) return pick_leaky_bwd<true, true>(a, s, used);
    if (wa) return pick_leaky_bwd<true, false>(a, s, used);
    if (ws) return pick_leaky_bwd<false, true>(a, s, used);
    return pick_leaky_bwd<false, false>(a, s, used);
}

bool tma_enabled()
{
    static const bool on = []() {
        const char *v = getenv("EXB_DISABLE_TMA");
        return !(v && v[0] == '1');
    }();
    return on;
}

// Reads and clears the status word of the current device (synchronises `stream`).
cudaError_t read_device_status(cudaStream_t s, unsigned int *out)
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
