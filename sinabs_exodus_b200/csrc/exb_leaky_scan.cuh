// Time-parallel leaky integrator (time-major layout) for long sequences with few neurons.
//
// The recurrence v_t = alpha*v_{t-1} + x_t is linear, so the time axis is cut into NSEG
// segments of L steps and every (neuron tile, segment) pair gets its own CTA:
//
//   pass A  integrate the segment from a zero state -> aggregate (the state it would end in)
//           and publish it to scratch memory with a ready flag
//   carry   wait (bounded) for the aggregates of all EARLIER segments of the tile and fold them
//           with Horner's rule:  carry <- alpha^L * carry + aggregate_i,  starting from v_init
//   pass B  integrate the segment again from the carry and write the results
//
// The segment is streamed twice through the same TMA ring; the second read is served by L2
// when the segments in flight fit there.  CTAs take their (segment, tile) from an atomic
// ticket, segment-major, so every CTA a waiting CTA depends on has already started; since
// pass A never waits, the aggregates always arrive.  Waits are bounded all the same.
//
// The backward pass is the same scan running from the end of time, with the alpha- and
// scale-gradient sums accumulated per segment in pass B and added to the outputs with
// atomicAdd (the launcher zeroes them first).
//
// Included by exb_tma_kernels.cu only (shares its status word and ring helpers).
#pragma once

namespace exb {

constexpr int SCAN_MAX_SEGMENTS = 64;

// Scratch memory layout (all offsets in 4-byte words):
//   [0]                       ticket counter
//   [1]                       number of CTAs that have finished
//   [16 .. 16+ntiles*nseg)    ready flags
//   [agg_off ..)              aggregates, ntiles*nseg*W floats
// The counters and flags must be zero when a launch starts.  The CTA that finishes last puts them back to
// zero, so a workspace that was zero once stays usable launch after launch without a memset in between
// (launches that share it must be ordered on one stream).
struct ScanWs {
    unsigned int *ticket;
    unsigned int *flags;
    float *agg;
};

struct ScanGeom {
    int nseg;      // segments per tile
    int L;         // steps per segment (multiple of the pipeline chunk tc)
    int ntiles;    // B * tiles_m
};

__host__ __device__ inline size_t scan_ws_words(int ntiles, int nseg, int W)
{
    const size_t flags = ((size_t)ntiles * nseg + 15) / 16 * 16;
    return 16 + flags + (size_t)ntiles * nseg * W;
}

__device__ __forceinline__ unsigned int ld_acquire(const unsigned int *p)
{
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_release(unsigned int *p, unsigned int v)
{
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// Diagnostic switch (exb_set_wait_limit): when non-zero no segment raises its ready flag, so every
// dependent segment's bounded wait runs out.  It exists so that the give-up path (status word, NaN
// poisoning, orderly return) can be exercised without any fault; it is 0 unless a test sets it.
static __constant__ unsigned int c_exb_scan_withhold_flags = 0u;

// Bounded spin on a ready flag written by another CTA of the same launch.
__device__ __forceinline__ bool wait_flag(const unsigned int *p)
{
    if (ld_acquire(p) != 0u) return true;
    const uint32_t limit = c_exb_wait_limit;
    for (uint32_t i = 1; i < limit; ++i) {
        __nanosleep(64);
        if (ld_acquire(p) != 0u) return true;
    }
    return false;
}

// alpha^n rounded once from double.
__device__ __forceinline__ float pow_int(float alpha, int n)
{
    double r = 1.0, a = (double)alpha;
    while (n > 0) {
        if (n & 1) r *= a;
        a *= a;
        n >>= 1;
    }
    return (float)r;
}

// Called by every thread of the CTA at the very end of a scan kernel (after ring_finish): the last CTA of the
// grid to get here clears the ticket, the finish counter and the ready flags for the next launch.  Everybody
// who read a flag has finished by then, since they count themselves in only after their last read.
__device__ __forceinline__ void scan_workspace_release(const ScanWs &ws, Ring *ring, int nflags)
{
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned int done = atomicAdd(ws.ticket + 1, 1u);
        ring->ticket = (done + 1u == gridDim.x) ? 1u : 0u;
    }
    __syncthreads();
    if (ring->ticket) {
        for (int i = threadIdx.x; i < nflags; i += blockDim.x) ws.flags[i] = 0u;
        if (threadIdx.x == 0) { ws.ticket[0] = 0u; ws.ticket[1] = 0u; }
    }
}

__device__ __forceinline__ void consumer_barrier(int nthreads)
{
    asm volatile("bar.sync 1, %0;" ::"r"(nthreads) : "memory");
}

// Producer for the two passes over one segment.  Pipeline op k (0 <= k < nA + nB) loads the
// box starting at time y(k); pass A ops load only tensor 0, pass B ops load all `nmaps`.
template <int NW, int V>
__device__ __forceinline__ void produce_segment(Ring *ring, float *stages, const CUtensorMap *const *maps, int nmaps,
                                                int nA, int nB, int t0, int m0, int b, PipeCfg pc, bool reverse)
{
    using G = TileGeom<NW, V>;
    const int tensor_floats = pc.tc * G::W;
    const int stage_floats = nmaps * tensor_floats;
    const int S = pc.stages;
    int k = 0;
    int s = 0;
    uint32_t par = 0u;             // (k / S) & 1, kept incrementally
    for (; k < nA + nB; ++k) {
        if (k >= S && !mbar_wait(smem_u32(&ring->empty[s]), par ^ 1u)) {
            report_timeout(EXB_STATUS_EMPTY_WAIT);
            ring->aborted = 1;
            break;
        }
        const bool passA = k < nA;
        const int idx = passA ? k : k - nA;                 // pipeline chunk inside the pass, in processing order
        const int nck = passA ? nA : nB;
        const int chunk = reverse ? (nck - 1 - idx) : idx;  // in time order
        const int nm = passA ? 1 : nmaps;
        const uint32_t bar = smem_u32(&ring->full[s]);
        mbar_arrive_expect_tx(bar, (uint32_t)(nm * tensor_floats * sizeof(float)));
        float *dst = stages + (size_t)s * stage_floats;
        for (int i = 0; i < nm; ++i) {
#pragma unroll
            for (int j = 0; j < G::NBOX; ++j)
                tma_load_3d(smem_u32(dst + i * tensor_floats + j * pc.tc * G::BW), maps[i], m0 + j * G::BW,
                            t0 + chunk * pc.tc, b, bar);
        }
        if (++s == S) { s = 0; par ^= 1u; }
    }
    ring->issued = k;
}

// Publishes the V values of this thread as the aggregate of (tile, seg) and raises the flag.
// A thread whose wait ran out still joins the barrier (so nobody is left waiting) but the flag
// stays down and the dependants give up after their own bounded wait.
template <int NW, int V>
__device__ __forceinline__ void publish_aggregate(const ScanWs &ws, Ring *ring, bool ok, int slot, int c,
                                                  const float (&y)[V])
{
    using G = TileGeom<NW, V>;
    float *dst = ws.agg + (size_t)slot * G::W + c;
    if (ok) {
#pragma unroll
        for (int j = 0; j < V; ++j) __stcg(dst + j, y[j]);
    }
    __threadfence();
    consumer_barrier(NW * 32);      // reached by every consumer thread, whatever `ok` is
    if (threadIdx.x == 0 && !ring->aborted && c_exb_scan_withhold_flags == 0u) st_release(ws.flags + slot, 1u);
}

// ---------------------------------------------------------------------------------------
template <int NW, int V>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V>::value)
leaky_fwd_scan_kernel(const __grid_constant__ TmaMaps maps, const LeakyFwdArgs A, const int tiles_m, const PipeCfg pc,
                      const ScanGeom sg, const ScanWs ws)
{
    using G = TileGeom<NW, V>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    const int tensor_floats = pc.tc * G::W;
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)pc.stages * tensor_floats * sizeof(float));
    if (threadIdx.x == 0) ring->ticket = atomicAdd(ws.ticket, 1u);
    ring_init(ring, pc.stages, NW);      // contains the __syncthreads that publishes the ticket
    const unsigned int s_ticket = ring->ticket;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (int)(s_ticket / (unsigned)sg.ntiles);      // segment-major ticket order
    const int tile = (int)(s_ticket % (unsigned)sg.ntiles);
    const int b = tile / tiles_m;
    const int m0 = (tile - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int t0 = seg * sg.L;
    const int nsteps = min(sg.L, T - t0);
    const int nck = (nsteps + pc.tc - 1) / pc.tc;
    const bool last_seg = (seg == sg.nseg - 1);
    const int nA = last_seg ? 0 : nck;      // nobody needs the aggregate of the last segment

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[1] = {&maps.m[0]};
            produce_segment<NW, V>(ring, stages, mp, 1, nA, nck, t0, m0, b, pc, false);
        }
    } else {
        const int c = threadIdx.x * V;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        float al[V], sc[V], v[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            al[j] = decay_of(A.alpha, b, mm + j);
            sc[j] = scale_of(A.scale, al[j], b, mm + j);
            v[j] = 0.0f;
        }
        const int64_t M = A.M;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        bool ok = true;
        RingPos pos = {0, 0u};
        int k = 0;
        // ---- pass A: aggregate from a zero state
        for (; k < nA; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *st = stages + (size_t)pos.s * tensor_floats + col;
            const int tmax = min(pc.tc, nsteps - k * pc.tc);
#pragma unroll 4
            for (int tt = 0; tt < tmax; ++tt) {
                float xs[V];
                lds_vec<V>(xs, st + tt * G::BW);
#pragma unroll
                for (int j = 0; j < V; ++j) v[j] = __fmaf_rn(v[j], al[j], __fmul_rn(sc[j], xs[j]));
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (nA > 0) publish_aggregate<NW, V>(ws, ring, ok, tile * sg.nseg + seg, c, v);
        // ---- carry: v_init folded with the aggregates of all earlier segments
#pragma unroll
        for (int j = 0; j < V; ++j) v[j] = A.v_init ? __ldg(A.v_init + n + j) : 0.0f;
        if (ok && seg > 0) {
            float aL[V];
#pragma unroll
            for (int j = 0; j < V; ++j) aL[j] = pow_int(al[j], sg.L);
            for (int i = 0; i < seg && ok; ++i) {
                const int slot = tile * sg.nseg + i;
                if (!wait_flag(ws.flags + slot)) {
                    report_timeout(EXB_STATUS_LOOKBACK_WAIT);
                    ring->aborted = 1;
                    ok = false;
                    break;
                }
                const float *src = ws.agg + (size_t)slot * G::W + c;
#pragma unroll
                for (int j = 0; j < V; ++j) v[j] = __fmaf_rn(v[j], aL[j], __ldcg(src + j));
            }
        }
        // ---- pass B: the real thing
        double total = 0.0;
        float *out = A.out + ((int64_t)b * T + t0) * M + mm;
        for (int kb = 0; kb < nck && ok; ++kb, ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *st = stages + (size_t)pos.s * tensor_floats + col;
            const int tmax = min(pc.tc, nsteps - kb * pc.tc);
            float part = 0.0f;
#pragma unroll 4
            for (int tt = 0; tt < tmax; ++tt) {
                float xs[V];
                lds_vec<V>(xs, st + tt * G::BW);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    v[j] = __fmaf_rn(v[j], al[j], __fmul_rn(sc[j], xs[j]));
                    part += v[j];
                }
                if (valid) stv<V>(out, v);
                out += M;
            }
            total += (double)part;
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        // The last segment depends on every other one: if any wait ran out, its own did too, and the
        // state it leaves is NaN so that the failure cannot go unnoticed downstream.
        if (valid && last_seg && A.v_last) {
#pragma unroll
            for (int j = 0; j < V; ++j) A.v_last[n + j] = ok ? v[j] : NAN;
        }
        if (A.out_sum) warp_add_f64(A.out_sum, valid ? (ok ? total : (double)NAN) : 0.0, lane);
    }
    ring_finish(ring, pc.stages);
    scan_workspace_release(ws, ring, sg.ntiles * sg.nseg);
}

// ---------------------------------------------------------------------------------------
// Backward: G_t = alpha*G_{t+1} + go_t scanned from the end of time.  Segment index `seg`
// counts in scan order; its time segment is q = nseg-1-seg, covering [q*L, min(T,(q+1)*L)).
template <int NW, int V>
__global__ void __launch_bounds__((NW + 1) * 32, MinBlocks<NW, V>::value)
leaky_bwd_scan_kernel(const __grid_constant__ TmaMaps maps, const LeakyBwdArgs A, const int tiles_m, const int nmaps,
                      const PipeCfg pc, const ScanGeom sg, const ScanWs ws, const bool WA, const bool WS)
{
    using G = TileGeom<NW, V>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    float *stages = reinterpret_cast<float *>(smem_raw);
    const int tensor_floats = pc.tc * G::W;
    const int stage_floats = nmaps * tensor_floats;
    Ring *ring = reinterpret_cast<Ring *>(smem_raw + (size_t)pc.stages * stage_floats * sizeof(float));
    if (threadIdx.x == 0) ring->ticket = atomicAdd(ws.ticket, 1u);
    ring_init(ring, pc.stages, NW);
    const unsigned int s_ticket = ring->ticket;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int seg = (int)(s_ticket / (unsigned)sg.ntiles);
    const int tile = (int)(s_ticket % (unsigned)sg.ntiles);
    const int q = sg.nseg - 1 - seg;
    const int b = tile / tiles_m;
    const int m0 = (tile - b * tiles_m) * G::W;
    const int T = (int)A.T;
    const int t0 = q * sg.L;
    const int nsteps = min(sg.L, T - t0);
    const int nck = (nsteps + pc.tc - 1) / pc.tc;
    const bool first_in_time = (q == 0);
    const int nA = first_in_time ? 0 : nck;   // the segment at t = 0 is last in scan order
    const int i_x = WA ? 2 : 1;

    if (warp == NW) {
        if (lane == 0) {
            const CUtensorMap *mp[5] = {&maps.m[0], &maps.m[1], &maps.m[2], &maps.m[3], &maps.m[4]};
            produce_segment<NW, V>(ring, stages, mp, nmaps, nA, nck, t0, m0, b, pc, true);
        }
    } else {
        const int c = threadIdx.x * V;
        const int64_t m = (int64_t)m0 + c;
        const bool valid = m < A.M;
        const int64_t mm = valid ? m : 0;
        const int64_t n = (int64_t)b * A.M + mm;
        float al[V], sc[V], Gv[V], glast[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            al[j] = decay_of(A.alpha, b, mm + j);
            sc[j] = scale_of(A.scale, al[j], b, mm + j);
            Gv[j] = 0.0f;
            glast[j] = A.g_last ? __ldg(A.g_last + n + j) : 0.0f;
        }
        const int64_t M = A.M;
        const int col = tile_col_off<NW, V>(pc.tc, c);
        bool ok = true;
        RingPos pos = {0, 0u};
        int k = 0;
        // ---- pass A: aggregate (value at the first step of the segment) from a zero carry
        for (; k < nA; ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *stg = stages + (size_t)pos.s * stage_floats + col;
            const int chunk = nck - 1 - k;
            const int tmax = min(pc.tc, nsteps - chunk * pc.tc);
#pragma unroll 4
            for (int tt = tmax - 1; tt >= 0; --tt) {
                float go[V];
                lds_vec<V>(go, stg + tt * G::BW);
                const bool last = (t0 + chunk * pc.tc + tt == T - 1);
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (last) go[j] = __fadd_rn(go[j], glast[j]);
                    Gv[j] = __fmaf_rn(Gv[j], al[j], go[j]);
                }
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        if (nA > 0) publish_aggregate<NW, V>(ws, ring, ok, tile * sg.nseg + seg, c, Gv);
        // ---- carry from all later time segments (earlier in scan order); they all have L steps
        // except the one at the end of time, whose own carry is zero.
#pragma unroll
        for (int j = 0; j < V; ++j) Gv[j] = 0.0f;
        if (ok && seg > 0) {
            float aL[V];
#pragma unroll
            for (int j = 0; j < V; ++j) aL[j] = pow_int(al[j], sg.L);
            for (int i = 0; i < seg && ok; ++i) {
                const int slot = tile * sg.nseg + i;
                if (!wait_flag(ws.flags + slot)) {
                    report_timeout(EXB_STATUS_LOOKBACK_WAIT);
                    ring->aborted = 1;
                    ok = false;
                    break;
                }
                const float *src = ws.agg + (size_t)slot * G::W + c;
#pragma unroll
                for (int j = 0; j < V; ++j) Gv[j] = __fmaf_rn(Gv[j], aL[j], __ldcg(src + j));
            }
        }
        // ---- pass B
        float ag[V], sgr[V];
#pragma unroll
        for (int j = 0; j < V; ++j) { ag[j] = 0.0f; sgr[j] = 0.0f; }
        float *gi_base = A.grad_input + ((int64_t)b * T + t0) * M + mm;
        for (int kb = 0; kb < nck && ok; ++kb, ++k) {
            if (!wait_chunk(ring, pos)) { ok = false; break; }
            const float *stg = stages + (size_t)pos.s * stage_floats + col;
            const int chunk = nck - 1 - kb;
            const int tmax = min(pc.tc, nsteps - chunk * pc.tc);
            float *gi = gi_base + (int64_t)(chunk * pc.tc + tmax - 1) * M;
#pragma unroll 4
            for (int tt = tmax - 1; tt >= 0; --tt) {
                const float *e = stg + tt * G::BW;
                float go[V], vo[V] = {}, xx[V] = {};
                lds_vec<V>(go, e);
                if (WA) lds_vec<V>(vo, e + tensor_floats);
                if (WS) lds_vec<V>(xx, e + i_x * tensor_floats);
                const bool last = (t0 + chunk * pc.tc + tt == T - 1);
                float r[V];
#pragma unroll
                for (int j = 0; j < V; ++j) {
                    if (last) go[j] = __fadd_rn(go[j], glast[j]);
                    if (WA) ag[j] = __fmaf_rn(Gv[j], vo[j], ag[j]);        // G_{t+1} * v_t
                    Gv[j] = __fmaf_rn(Gv[j], al[j], go[j]);
                    if (WS) sgr[j] = __fmaf_rn(Gv[j], xx[j], sgr[j]);
                    r[j] = __fmul_rn(sc[j], Gv[j]);
                }
                if (valid) stv<V>(gi, r);
                gi -= M;
            }
            release_chunk(ring, pos, lane);
            pos.advance(pc.stages);
        }
        float gdecay[V];
#pragma unroll
        for (int j = 0; j < V; ++j) {
            gdecay[j] = 0.0f;
            if (valid) {
                if (!ok) { ag[j] = NAN; sgr[j] = NAN; Gv[j] = NAN; }      // gave up: poison what depends on this segment
                if (first_in_time) {
                    if (A.grad_init) A.grad_init[n + j] = __fmul_rn(al[j], Gv[j]);
                    if (WA) ag[j] = __fmaf_rn(Gv[j], A.v_init ? __ldg(A.v_init + n + j) : 0.0f, ag[j]);
                }
                if (A.acc_decay) {      // this segment's share; the chain rule is linear in it
                    gdecay[j] = decay_param_grad(ag[j], sgr[j], A.alpha, A.scale, al[j], b, mm + j);
                } else {
                    if (WA) atomicAdd(A.grad_alpha + n + j, ag[j]);
                    if (WS) atomicAdd(A.grad_scale + n + j, sgr[j]);
                }
            }
        }
        if (A.acc_decay) acc_param_grad<V>(A.acc_decay, A.alpha, gdecay, valid, b, mm, lane);
    }
    ring_finish(ring, pc.stages);
    scan_workspace_release(ws, ring, sg.ntiles * sg.nseg);
}

}  // namespace exb
