// The small stages between the weight-streaming GEMVs: activation staging
// (RMSNorm + quantisation), the router, the expert activation, and the partial-sum
// reduction with the in-kernel tensor-parallel all-reduce.
//
// Reference counterparts: glm53/gfx950/kernel.py:1367-1414 (RMSNorm staging),
// :1440-1466 (quant_scaled / quant_mxfp8), :1575-1629 (route_top8), :4396-4415 (SiLU),
// :1631-1688 (peer_reduce); minimax_m31/ffn.py:601-723 (router).
#include <cooperative_groups.h>
#include <cstdlib>
#include "mono_common.cuh"
#include "rowdot.cuh"
#include "act_quant.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {

// ------------------------------------------------------------------ act_prep
// One CTA per row.  The row is staged in shared memory as f32, normalised, then
// quantised one 128-chunk per warp.
// Launch bounds of the small stage kernels name a minimum block count on purpose: with the thread count alone
// the compiler settles on 32 registers per thread (full occupancy), spills, and waits for each load of a batch
// before issuing the next.  These kernels run a handful of blocks and live on memory round trips: registers
// for a whole batch of loads in flight are worth more than occupancy they never use.
constexpr int kPrepThreads = 1024;

// The part of the staging after a row is in shared memory as f32 (and `ssq` holds this thread's share of its
// sum of squares): RMSNorm, bf16 rounding, the plain bf16 copy, the quantised planes.
__device__ __forceinline__ void prep_tail(const mono_act_prep_args& a, int row, int seg, int segs, float* xrow, float* red, float ssq) {
    const int tid = threadIdx.x;
    if (a.gamma_bf16) {
        const __nv_bfloat16* gm = reinterpret_cast<const __nv_bfloat16*>(a.gamma_bf16);
        uint2 graw[4];  // gamma is fetched before the reduction so that its latency hides behind it
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = tid * 4 + j * kPrepThreads * 4;
            graw[j] = i < a.k ? __ldg(reinterpret_cast<const uint2*>(gm + i)) : make_uint2(0, 0);
        }
        const float tot = block_sum<kPrepThreads / 32>(ssq, red);
        const float r = rsqrtf(tot / (float)a.k + a.eps);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = tid * 4 + j * kPrepThreads * 4;
            if (i < a.k) {
                const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw[j].x));
                const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw[j].y));
                float4 v = *reinterpret_cast<float4*>(xrow + i);
                v.x = v.x * r * lo.x; v.y = v.y * r * lo.y; v.z = v.z * r * hi.x; v.w = v.w * r * hi.y;
                *reinterpret_cast<float4*>(xrow + i) = v;
            }
        }
    }
    __syncthreads();
    if (a.round_bf16)
        for (int i = tid; i < a.k; i += kPrepThreads) xrow[i] = bf16_round(xrow[i]);
    __syncthreads();
    if (a.out_bf16) {
        __nv_bfloat16* o = reinterpret_cast<__nv_bfloat16*>(a.out_bf16) + ((size_t)row * segs + seg) * a.k;
        for (int i = tid; i < a.k; i += kPrepThreads) o[i] = __float2bfloat16_rn(xrow[i]);
    }
    if (a.planes) {
        const int warp = tid >> 5, lane = tid & 31;
        uint8_t* p0 = a.planes + (size_t)seg * a.seg_stride + (size_t)row * a.ld;
        uint8_t* p1 = p0 + a.plane_stride;
        float* sf = a.scale_f32 ? a.scale_f32 + (size_t)seg * a.scale_seg_stride + (size_t)row * a.scale_ld : nullptr;
        uint8_t* s8 = a.scale_e8 ? a.scale_e8 + (size_t)seg * a.scale_seg_stride + (size_t)row * a.scale_ld : nullptr;
        for (int c = warp; c < a.k / 128; c += kPrepThreads / 32) quant_chunk128(xrow + c * 128, a.fmt, lane, c, p0, p1, sf, s8);
    }
}

__global__ void __launch_bounds__(kPrepThreads, 1) act_prep_kernel(const mono_act_prep_args a) {
    pdl_launch_dependents();
    prefetch_span(a.gamma_bf16, (size_t)a.k * 2, threadIdx.x, kPrepThreads);  // the norm weights, during the wait
    pdl_wait();
    extern __shared__ float xrow[];
    __shared__ float red[kPrepThreads / 32];
    const int segs = a.segs > 1 ? a.segs : 1;
    const int row = blockIdx.x / segs, seg = blockIdx.x - row * segs, tid = threadIdx.x;
    // four values per thread per pass, every load of a pass issued before it is used:
    // the row arrives in one or two memory latencies instead of one per element
    float ssq = 0.f;
    for (int i = tid * 4; i < a.k; i += kPrepThreads * 4) {
        float4 v;
        if (a.src_bf16) {
            const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.src_bf16) +
                                                              ((size_t)row * segs + seg) * a.k + i);
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            v = make_float4(lo.x, lo.y, hi.x, hi.y);
        } else {
            v = sum_partials4<8>(a.src_f32 + (size_t)row * a.src_ld + (size_t)seg * a.k + i, a.src_sum_stride, a.nsum);
        }
        *reinterpret_cast<float4*>(xrow + i) = v;
        ssq += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    prep_tail(a, row, seg, segs, xrow, red, ssq);
}

// ------------------------------------------------------------------ router
// One CTA, one warp per row.  Picks are exact on the stored f32 scores: key =
// monotone image of (score + bias), ties to the lower expert id.
constexpr int kRouteThreads = 512;
constexpr int kMaxExperts = 512;

__device__ __forceinline__ uint32_t radix_key(float f) {
    uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b ^ 0x80000000u);
}

// The routing of one step by one CTA of kRouteThreads threads, one warp per row.  A single CTA runs
// this code once, so what it costs is the instructions it has to fetch: the loops stay rolled,
// the row's logits arrive by one batch of asynchronous copies, and the picks scan shared memory.
struct RouteSmem {
    float sc[kMaxRows][kMaxExperts];
    float bias[kMaxExperts];
    int used[kMaxExperts];
    int sel[kMaxRows][16];
    float selw[kMaxRows][16];
    int slot_of[kMaxExperts];
    int warp_cnt[kRouteThreads / 32];
};

template <int kSlots>  // experts per lane: 8 serves up to 256 experts, 16 up to 512
__device__ __forceinline__ void route_body(const mono_route_args& a, RouteSmem& sm) {
    auto& sc = sm.sc;
    auto& used = sm.used;
    auto& sel = sm.sel;
    auto& selw = sm.selw;
    auto& slot_of = sm.slot_of;
    auto& warp_cnt = sm.warp_cnt;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // the logits may come from other CTAs of this launch: they are copied past L1 (16-byte
    // asynchronous copies, all in flight together), or read with ld.cg where that shape does not fit
    const bool vec = a.nsum == 1 && !(a.ld & 3) && !(a.n_experts & 3) && !(reinterpret_cast<uintptr_t>(a.logits) & 15);
    if (vec && warp < a.rows) {
#pragma unroll 1
        for (int c = lane; c < a.n_experts / 4; c += 32)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(&sc[warp][4 * c])),
                         "l"(a.logits + (size_t)warp * a.ld + 4 * c)
                         : "memory");
    }
#pragma unroll 1
    for (int e = tid; e < a.n_experts; e += kRouteThreads) {
        used[e] = 0;
        sm.bias[e] = a.bias ? __ldg(a.bias + e) : 0.f;
    }
    asm volatile("cp.async.wait_all;" ::: "memory");
    __syncthreads();
    if (warp < a.rows) {
        const int r = warp;
        const bool live = !a.slots || a.slots[r] >= 0;
#pragma unroll 1
        for (int e = lane; e < a.n_experts; e += 32) {
            float l = 0.f;
            if (vec) {
                l = sc[r][e];
            } else {
                for (int p = 0; p < a.nsum; ++p) l += __ldcg(a.logits + (size_t)p * a.sum_stride + (size_t)r * a.ld + e);
            }
            const float s = 1.f / (1.f + expf(-l));
            sc[r][e] = s;
            if (a.scores) a.scores[(size_t)r * a.n_experts + e] = s;
        }
        __syncwarp();
        // a lane owns experts lane, lane + 32, ... and keeps their keys (monotone image of score + bias;
        // 0 = none, or already picked) in kSlots registers.  A pick = the largest key of the warp, then the
        // lowest expert id among its holders (a lane's lowest id is its lowest slot: the first strict
        // maximum).  The loop over the picks stays rolled; only the kSlots-wide steps inside are unrolled.
        uint32_t keys[kSlots];
#pragma unroll
        for (int i = 0; i < kSlots; ++i) {
            const int e = lane + 32 * i;
            keys[i] = 0u;
            if (e < a.n_experts) keys[i] = radix_key(a.bias ? sc[r][e] + sm.bias[e] : sc[r][e]);
        }
        float wsum = 0.f;
#pragma unroll 1
        for (int k = 0; k < a.top_k; ++k) {
            uint32_t best = 0u;
            int slot = 0;
#pragma unroll
            for (int i = 0; i < kSlots; ++i)
                if (keys[i] > best) { best = keys[i]; slot = i; }
            const uint32_t top = __reduce_max_sync(0xffffffffu, best);
            const int e = (int)__reduce_min_sync(0xffffffffu, best == top ? (uint32_t)(lane + 32 * slot) : 0xFFFFFFFFu);
#pragma unroll
            for (int i = 0; i < kSlots; ++i)
                if (lane == (e & 31) && i == (e >> 5)) keys[i] = 0u;
            if (lane == 0) { sel[r][k] = e; selw[r][k] = sc[r][e]; }
            wsum += sc[r][e];
        }
        __syncwarp();
        const float norm = a.route_scale / fmaxf(wsum, 1e-20f);
        if (lane < a.top_k) {
            const int e = live ? sel[r][lane] : -1;
            const float w = live ? selw[r][lane] * norm : 0.f;
            a.ids[r * a.top_k + lane] = e;
            a.weights[r * a.top_k + lane] = w;
            sel[r][lane] = e;
            selw[r][lane] = w;
            if (live) used[e] = 1;
        }
    }
    __syncthreads();
    // distinct experts in ascending id: ordered compaction
    int flag = 0;
    if (tid < a.n_experts) flag = used[tid];
    const unsigned bal = __ballot_sync(0xffffffffu, flag);
    if (lane == 0) warp_cnt[warp] = __popc(bal);
    __syncthreads();
    int base = 0;
    for (int w = 0; w < warp; ++w) base += warp_cnt[w];
    if (tid < a.n_experts) slot_of[tid] = flag ? base + __popc(bal & ((1u << lane) - 1)) : -1;
    __syncthreads();
    int total = 0;
    for (int w = 0; w < kRouteThreads / 32; ++w) total += warp_cnt[w];
    if (tid < a.n_experts && flag) a.expert_list[slot_of[tid]] = tid;
    if (tid == 0) *a.n_expert = total;
    for (int i = tid; i < total * kMaxRows; i += kRouteThreads) a.coef[i] = 0.f;
    __syncthreads();
    if (tid < a.rows * a.top_k) {
        const int r = tid / a.top_k, k = tid - r * a.top_k;
        const int e = sel[r][k];
        if (e >= 0) a.coef[slot_of[e] * kMaxRows + r] = selw[r][k];
    }
}

__global__ void __launch_bounds__(kRouteThreads, 1) route_kernel(const mono_route_args a) {
    __shared__ RouteSmem sm;
    pdl_launch_dependents();
    prefetch_span(a.bias, (size_t)a.n_experts * 4, threadIdx.x, kRouteThreads);  // during the wait for the logits
    pdl_wait();
    if (a.n_experts <= 256) route_body<8>(a, sm);
    else route_body<16>(a, sm);
}

template <int COLS, bool STAGED>
__global__ void __launch_bounds__(kRowdotThreads, 1) rowdot_kernel(const mono_rowdot_args a) {
    // one CTA per COLS output columns; STAGED: the launch has rows x k bf16 of dynamic shared memory for the rows
    extern __shared__ __align__(16) uint8_t rowdot_xs[];
    __shared__ float red[COLS][kRowdotThreads / 32][kMaxRows];
    pdl_launch_dependents();
    MONO_TL(tl_rowdot, 0);
    rowdot_col<COLS, STAGED>(a, blockIdx.x * COLS, threadIdx.x, red, reinterpret_cast<const __nv_bfloat16*>(rowdot_xs));
}

// Router logits and routing in one launch: every CTA computes two columns of the logits (one per
// group of 256 threads, the arithmetic of rowdot_kernel), and the CTA that finishes last routes the
// step.  No CTA waits for another: the last one is known from a counter, which it puts back to zero.
constexpr int kRouterCols = kRouteThreads / kRowdotThreads;

__global__ void __launch_bounds__(kRouteThreads) router_kernel(const mono_rowdot_args d, const mono_route_args r, int32_t* counter) {
    __shared__ float red[kRouterCols][1][kRowdotThreads / 32][kMaxRows];
    __shared__ RouteSmem sm;
    __shared__ int is_last;
    pdl_launch_dependents();
    const int group = threadIdx.x / kRowdotThreads, t = threadIdx.x - group * kRowdotThreads;
    rowdot_col<1>(d, blockIdx.x * kRouterCols + group, t, red[group]);
    __threadfence();  // this CTA's logits are visible device-wide before it is counted
    __syncthreads();
    if (threadIdx.x == 0) {
        const int prev = atomicAdd(counter, 1);
        is_last = prev == (int)gridDim.x - 1;
        if (is_last) *counter = 0;  // every CTA of this launch has been counted
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (r.n_experts <= 256) route_body<8>(r, sm);
    else route_body<16>(r, sm);
}

// ------------------------------------------------------------------ expert activation
constexpr int kMidThreads = 256;

__device__ __forceinline__ void mid_body(const mono_mid_args& a, int block, float (*chunk)[128]) {
    const int slot = block / a.rows, row = block - slot * a.rows;
    const int nslot = a.n_slot ? min(*a.n_slot, a.max_slot) : a.max_slot;
    if (slot >= nslot) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const size_t ld2 = 2 * (size_t)a.inter;
    const float* up = a.up + ((size_t)slot * a.nsum * kMaxRows + row) * ld2;
    const size_t sum_stride = (size_t)kMaxRows * ld2;
    const int ld_bytes = a.ld;
    uint8_t* p0 = a.planes + ((size_t)slot * kMaxRows + row) * ld_bytes;
    float* sf = a.scale_f32 ? a.scale_f32 + ((size_t)slot * kMaxRows + row) * a.scale_ld : nullptr;
    uint8_t* s8 = a.scale_e8 ? a.scale_e8 + ((size_t)slot * kMaxRows + row) * a.scale_ld : nullptr;
    for (int c = warp; c < a.inter / 128; c += kMidThreads / 32) {
        const float* gp = up + c * 128 + 4 * lane;
        const float4 g4 = sum_partials4<4>(gp, sum_stride, a.nsum), u4 = sum_partials4<4>(gp + a.inter, sum_stride, a.nsum);
        const float gs[4] = {g4.x, g4.y, g4.z, g4.w}, us[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            float m = gs[i] / (1.f + expf(-gs[i])) * us[i];
            if (a.round_bf16) m = bf16_round(m);
            chunk[warp][4 * lane + i] = m;
        }
        __syncwarp();
        quant_chunk128(chunk[warp], a.fmt, lane, c, p0, nullptr, sf, s8);
        __syncwarp();
    }
}

__global__ void __launch_bounds__(kMidThreads, 4) mid_kernel(const mono_mid_args a) {
    pdl_prologue();
    __shared__ float chunk[kMidThreads / 32][128];
    mid_body(a, blockIdx.x, chunk);
}

// Two activation stages in one launch (the shared expert's and the routed experts'): blocks
// [0, a.max_slot * a.rows) serve `a`, the rest `b`.
__global__ void __launch_bounds__(kMidThreads, 4) mid_pair_kernel(const mono_mid_args a, const mono_mid_args b) {
    pdl_prologue();
    __shared__ float chunk[kMidThreads / 32][128];
    const int na = a.max_slot * a.rows;
    if ((int)blockIdx.x < na) mid_body(a, blockIdx.x, chunk);
    else mid_body(b, blockIdx.x - na, chunk);
}

// ------------------------------------------------------------------ reduce + all-reduce
// Every thread owns one bf16 pair (two adjacent columns) of one row.
constexpr int kReduceThreads = 256;

__device__ __forceinline__ void st_sys_v2(uint64_t addr, uint32_t a, uint32_t b) {
    asm volatile("st.relaxed.sys.global.v2.u32 [%0], {%1,%2};" ::"l"(addr), "r"(a), "r"(b) : "memory");
}
__device__ __forceinline__ uint2 ld_sys_v2(uint64_t addr) {
    uint2 v;
    asm volatile("ld.relaxed.sys.global.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(addr) : "memory");
    return v;
}
// One store that the switch delivers to every rank's copy of a multicast-bound buffer (NVLS).
__device__ __forceinline__ void st_multimem_v2(uint64_t mc_addr, uint32_t a, uint32_t b) {
    const uint64_t v = (uint64_t)a | ((uint64_t)b << 32);
    asm volatile("multimem.st.relaxed.sys.global.b64 [%0], %1;" ::"l"(mc_addr), "l"(v) : "memory");
}
__device__ __forceinline__ void st_sys_u32(uint64_t addr, uint32_t a) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(addr), "r"(a) : "memory");
}

// Waits for the (value, tag) word at `addr` of this rank's own peer region to carry `tag`.  Every 64 polls
// it looks at the sticky error words and the peers' flag words and at the deadline (common/sync.py:31-98,
// common/guard.py:100-241): a wait that runs out stores site + 1 in the deadline word and raises this
// rank's flag at every peer; a wait that sees a failure elsewhere gives up at once.  *failed says which.
__device__ __forceinline__ uint2 poll_tagged(uint64_t addr, uint32_t tag, int32_t* guard, const uint64_t* peer_guards, int world,
                                             int rank, int site, uint64_t deadline_ns, uint64_t t0, bool* failed) {
    uint2 v = ld_sys_v2(addr);
    uint32_t spins = 0;
    while (v.y != tag) {
        if ((++spins & 63) == 0) {
            if (guard_failed(guard)) { *failed = true; break; }
            const volatile int* gw = guard;
            if (gw) {
                for (int r = 0; r < world; ++r)
                    if (gw[MONO_GUARD_FLAGS + r]) { guard_fail(guard, MONO_ERR_PEER, r); *failed = true; }
                if (*failed) break;
            }
            if (globaltimer_ns() - t0 > deadline_ns) {
                guard_fail(guard, MONO_ERR_DEADLINE, site);
                if (peer_guards)
                    for (int d = 0; d < world; ++d)
                        if (d != rank) st_sys_u32(peer_guards[d] + 4ull * (MONO_GUARD_FLAGS + rank), 1u);
                *failed = true;
                break;
            }
        }
        v = ld_sys_v2(addr);
    }
    return v;
}

// One pair of columns of one row through the ranks: `word` is this rank's bf16 partial, (res0, res1) the residual;
// returns the finished bf16 pair (rank-ordered f32 sum + residual).  Two forms with the same arithmetic and bits:
//   all-to-all   every rank pushes its word to every rank and sums the `world` words it received;
//   rs + ag      (a.rsag; minimax_m3/gfx950/layout.py:33-34,97-114: "half the bytes a link, one more hop") the rank
//                that owns the pair's column slice receives the words, sums them, adds the residual and pushes the
//                FINISHED word to the others, which only wait for it.  The finished word travels in the slot the
//                all-to-all form uses for the owner's partial: in a peer's buffer that slot's columns are free,
//                because a rank sends a peer partials of the peer's own slice only.
__device__ __forceinline__ uint32_t exchange_pair(const mono_reduce_args& a, int row, int pc, int pairs, uint32_t word, uint32_t tag,
                                                  int parity, float res0, float res1, uint64_t t0, bool* failed) {
    const size_t slot_pairs = (size_t)kMaxRows * pairs;
    const size_t row_off = (size_t)row * pairs + pc;
    const size_t my_off = (((size_t)parity * a.world + a.rank) * slot_pairs + row_off) * 8;
    const uint64_t mine = a.peer_ptrs[a.rank];
    const int owner = a.rsag ? pc / (pairs / a.world) : a.rank;
    if (!a.rsag) {
        if (a.mc_ptr) st_multimem_v2(a.mc_ptr + my_off, word, tag);
        else
            for (int d = 0; d < a.world; ++d) st_sys_v2(a.peer_ptrs[d] + my_off, word, tag);
    } else {
        st_sys_v2(a.peer_ptrs[owner] + my_off, word, tag);
    }
    *failed = *failed || guard_failed(a.guard);
    if (owner != a.rank) {  // rs + ag, somebody else's slice: the finished word arrives in the owner's slot
        const uint64_t addr = mine + (((size_t)parity * a.world + owner) * slot_pairs + row_off) * 8;
        if (*failed) return 0u;
        return poll_tagged(addr, tag, a.guard, a.peer_guards, a.world, a.rank, a.site, a.deadline_ns, t0, failed).x;
    }
    float acc0 = 0.f, acc1 = 0.f;
    for (int src = 0; src < a.world && !*failed; ++src) {
        const uint64_t addr = mine + (((size_t)parity * a.world + src) * slot_pairs + row_off) * 8;
        const uint2 v = poll_tagged(addr, tag, a.guard, a.peer_guards, a.world, a.rank, a.site, a.deadline_ns, t0, failed);
        if (*failed) break;
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
        acc0 += __low2float(b);
        acc1 += __high2float(b);
    }
    const __nv_bfloat162 o = __floats2bfloat162_rn(acc0 + res0, acc1 + res1);
    const uint32_t ow = *reinterpret_cast<const uint32_t*>(&o);
    if (a.rsag && !*failed) {
        if (a.mc_ptr) st_multimem_v2(a.mc_ptr + my_off, ow, tag);
        else
            for (int d = 0; d < a.world; ++d)
                if (d != a.rank) st_sys_v2(a.peer_ptrs[d] + my_off, ow, tag);
    }
    return ow;
}

__global__ void __launch_bounds__(kReduceThreads, 2) reduce_kernel(const mono_reduce_args a) {
    pdl_launch_dependents();
    const int pairs = a.n / 2;
    const int total = a.rows * pairs;
    if (a.residual && (threadIdx.x & 31) == 0) {
        // during the wait for the GEMV before this launch: the residual pairs of this warp's first turn
        // (128 bytes; the residual is older than that GEMV's output)
        const int idx0 = blockIdx.x * kReduceThreads + threadIdx.x;
        if (idx0 < total) prefetch_l2(reinterpret_cast<const __nv_bfloat162*>(a.residual) + idx0);
    }
    pdl_wait();
    uint32_t tag = a.tag;
    int parity = a.parity;
    if (a.world > 1 && a.guard && tag == 0) {
        const int epoch = reinterpret_cast<const volatile int*>(a.guard)[MONO_GUARD_EPOCH];
        tag = (uint32_t)epoch * 256u + (uint32_t)a.site + 1u;
        parity = epoch & 1;
    }
    for (int idx = blockIdx.x * kReduceThreads + threadIdx.x; idx < total; idx += gridDim.x * kReduceThreads) {
        const int row = idx / pairs, pc = idx - row * pairs;
        const bool live = !a.slots || a.slots[row] >= 0;
        float p0 = 0.f, p1 = 0.f;
        if (live) {
            const float2 v = sum_partials2<8>(a.partial + (size_t)row * a.ld + 2 * pc, a.sum_stride, a.nsum);
            p0 = v.x;
            p1 = v.y;
        }
        __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        float res0 = 0.f, res1 = 0.f;
        if (a.residual) {
            const __nv_bfloat162 r = reinterpret_cast<const __nv_bfloat162*>(a.residual)[(size_t)row * pairs + pc];
            res0 = __low2float(r);
            res1 = __high2float(r);
        }
        uint32_t ow;
        if (a.world > 1) {
            bool failed = false;
            ow = exchange_pair(a, row, pc, pairs, *reinterpret_cast<uint32_t*>(&pb), tag, parity, res0, res1, globaltimer_ns(), &failed);
        } else {
            const __nv_bfloat162 o = __floats2bfloat162_rn(__low2float(pb) + res0, __high2float(pb) + res1);
            ow = *reinterpret_cast<const uint32_t*>(&o);
        }
        reinterpret_cast<uint32_t*>(a.out)[(size_t)row * pairs + pc] = ow;
    }
}

// The reduction of reduce_kernel and the staging of act_prep_kernel in one launch.  A cluster of C CTAs serves a
// row, CTA c its columns [c k / C, (c + 1) k / C): the partial slices are added in order, rounded to bf16, all-reduced
// over the ranks (pushes, bounded polls, sum in rank order), the residual is added and the bf16 result is written to
// r.out (element for element the arithmetic of reduce_kernel: same bits).  The same values then go through the norm
// and the quantisation of `a` (whose source fields are not read); the row's sum of squares is the C CTAs' sums added
// in CTA order, exchanged over distributed shared memory.  A thread waits for other GPUs' words only, and every
// CTA reaches both cluster barriers whatever its polls returned.
constexpr int kRnThreads = 256;

template <int C>
__global__ void __cluster_dims__(C, 1, 1) __launch_bounds__(kRnThreads, 1) reduce_norm_kernel(const mono_reduce_args r, const mono_act_prep_args a) {
    namespace cg = cooperative_groups;
    pdl_launch_dependents();
    cg::cluster_group cluster = cg::this_cluster();
    const int row = blockIdx.x / C, crank = (int)cluster.block_rank(), tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int kc = a.k / C, col0 = crank * kc;  // this CTA's columns (a multiple of 128)
    const int pairs = r.n / 2;
    if (a.gamma_bf16) prefetch_span(reinterpret_cast<const __nv_bfloat16*>(a.gamma_bf16) + col0, (size_t)kc * 2, tid, kRnThreads);
    if (r.residual) prefetch_span(reinterpret_cast<const __nv_bfloat16*>(r.residual) + (size_t)row * r.n + col0, (size_t)kc * 2, tid, kRnThreads);
    pdl_wait();
    extern __shared__ float xrow[];  // kc values
    __shared__ float red[kRnThreads / 32];
    __shared__ float cl_ssq;
    uint32_t tag = r.tag;
    int parity = r.parity;
    if (r.world > 1 && r.guard && tag == 0) {
        const int epoch = reinterpret_cast<const volatile int*>(r.guard)[MONO_GUARD_EPOCH];
        tag = (uint32_t)epoch * 256u + (uint32_t)r.site + 1u;
        parity = epoch & 1;
    }
    const bool live = !r.slots || r.slots[row] >= 0;
    const uint64_t t0 = r.world > 1 ? globaltimer_ns() : 0;
    float ssq = 0.f;
    for (int li = tid * 4; li < kc; li += kRnThreads * 4) {
        const int i = col0 + li;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live) {
            v = sum_partials4<8>(r.partial + (size_t)row * r.ld + i, r.sum_stride, r.nsum);  // slices added in order
        }
        const __nv_bfloat162 pb0 = __floats2bfloat162_rn(v.x, v.y), pb1 = __floats2bfloat162_rn(v.z, v.w);
        float2 rlo = make_float2(0.f, 0.f), rhi = rlo;
        if (r.residual) {
            const uint2 raw = *reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(r.residual) + (size_t)row * r.n + i);
            rlo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            rhi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
        }
        uint32_t ow0, ow1;
        if (r.world > 1) {
            const int pc = i >> 1;  // this thread's two pairs: pc, pc + 1
            bool failed = false;
            ow0 = exchange_pair(r, row, pc, pairs, *reinterpret_cast<const uint32_t*>(&pb0), tag, parity, rlo.x, rlo.y, t0, &failed);
            ow1 = exchange_pair(r, row, pc + 1, pairs, *reinterpret_cast<const uint32_t*>(&pb1), tag, parity, rhi.x, rhi.y, t0, &failed);
        } else {
            const __nv_bfloat162 q0 = __floats2bfloat162_rn(__low2float(pb0) + rlo.x, __high2float(pb0) + rlo.y);
            const __nv_bfloat162 q1 = __floats2bfloat162_rn(__low2float(pb1) + rhi.x, __high2float(pb1) + rhi.y);
            ow0 = *reinterpret_cast<const uint32_t*>(&q0);
            ow1 = *reinterpret_cast<const uint32_t*>(&q1);
        }
        const __nv_bfloat162 o0 = *reinterpret_cast<const __nv_bfloat162*>(&ow0), o1 = *reinterpret_cast<const __nv_bfloat162*>(&ow1);
        *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(r.out) + (size_t)row * r.n + i) = make_uint2(ow0, ow1);
        const float4 h = make_float4(__low2float(o0), __high2float(o0), __low2float(o1), __high2float(o1));
        *reinterpret_cast<float4*>(xrow + li) = h;
        ssq += h.x * h.x + h.y * h.y + h.z * h.z + h.w * h.w;
    }
    // ---- the row's sum of squares: this CTA's share, then the C shares in CTA order
    const float mine_ssq = block_sum<kRnThreads / 32>(ssq, red);
    if (tid == 0) cl_ssq = mine_ssq;
    cluster.sync();
    float rstd = 1.f;
    if (a.gamma_bf16) {
        float tot = 0.f;
#pragma unroll
        for (int c = 0; c < C; ++c) tot += *cluster.map_shared_rank(&cl_ssq, c);
        rstd = rsqrtf(tot / (float)a.k + a.eps);
    }
    for (int li = tid * 4; li < kc; li += kRnThreads * 4) {
        float4 v = *reinterpret_cast<float4*>(xrow + li);
        if (a.gamma_bf16) {
            const uint2 graw = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.gamma_bf16) + col0 + li));
            const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.x));
            const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&graw.y));
            v.x = v.x * rstd * lo.x; v.y = v.y * rstd * lo.y; v.z = v.z * rstd * hi.x; v.w = v.w * rstd * hi.y;
        }
        if (a.round_bf16) { v.x = bf16_round(v.x); v.y = bf16_round(v.y); v.z = bf16_round(v.z); v.w = bf16_round(v.w); }
        *reinterpret_cast<float4*>(xrow + li) = v;
        if (a.out_bf16) {
            const __nv_bfloat162 b0 = __floats2bfloat162_rn(v.x, v.y), b1 = __floats2bfloat162_rn(v.z, v.w);
            *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out_bf16) + (size_t)row * a.k + col0 + li) =
                make_uint2(*reinterpret_cast<const uint32_t*>(&b0), *reinterpret_cast<const uint32_t*>(&b1));
        }
    }
    __syncthreads();
    if (a.planes) {
        uint8_t* p0 = a.planes + (size_t)row * a.ld;
        uint8_t* p1 = p0 + a.plane_stride;
        float* sf = a.scale_f32 ? a.scale_f32 + (size_t)row * a.scale_ld : nullptr;
        uint8_t* s8 = a.scale_e8 ? a.scale_e8 + (size_t)row * a.scale_ld : nullptr;
        for (int c = warp; c < kc / 128; c += kRnThreads / 32) quant_chunk128(xrow + c * 128, a.fmt, lane, col0 / 128 + c, p0, p1, sf, s8);
    }
    cluster.sync();  // no CTA leaves while another may still read its sum
}

// Pulls up to MONO_PREFETCH_RANGES byte ranges towards L2 (cp.async.bulk.prefetch.L2, 16 KB a request).  A launch of
// its own on a side branch of the step's graph: weights that a later stage will stream do not depend on anything,
// and the stages between two weight streams leave HBM idle (they live on memory round trips, not on bandwidth).
// Nothing waits for these requests: the kernel only issues them.
__global__ void __launch_bounds__(128, 1) l2_prefetch_kernel(const mono_prefetch_args a) {
    pdl_launch_dependents();
    constexpr uint32_t kChunk = 16384;
    const long tid = (long)blockIdx.x * blockDim.x + threadIdx.x, nthreads = (long)gridDim.x * blockDim.x;
    for (int r = 0; r < a.n; ++r) {
        const uint8_t* base = reinterpret_cast<const uint8_t*>(a.ptr[r]);
        const long chunks = (long)((a.bytes[r] + kChunk - 1) / kChunk);
        for (long c = tid; c < chunks; c += nthreads) {
            const uint64_t left = a.bytes[r] - (uint64_t)c * kChunk;
            const uint32_t sz = (uint32_t)(left < kChunk ? (left & ~15ull) : kChunk);
            if (sz) asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(base + (uint64_t)c * kChunk), "r"(sz) : "memory");
        }
    }
}

__global__ void epoch_advance_kernel(int32_t* guard) {
    pdl_prologue();
    guard[MONO_GUARD_EPOCH] += 1;
}

// ------------------------------------------------------------------ LM-head logits: K-split sum + all-gather
// Every thread owns one pair of adjacent columns of one row of this rank's share of the vocabulary:
// it adds the K splits in order, and with world > 1 rounds the pair to bf16, stores (pair, tag) into every
// rank's logits region at [parity][row][rank * n_local / 2 + pair], then waits for the same pair of every
// other rank in its own region and widens it to f32 (glm53_flash/gfx950/kernel.py:3700-3770; two slots by
// launch parity, glm53_flash/gfx950/layout.py:193-215).  A thread waits for words of other GPUs only, never
// for another CTA of this launch, so the grid need not be resident at once.
__global__ void __launch_bounds__(kReduceThreads, 2) logits_gather_kernel(const mono_logits_gather_args a) {
    pdl_prologue();
    const int pairs = a.n_local / 2;
    const int total = a.rows * pairs;
    const int all_pairs = a.world * pairs;
    uint32_t tag = a.tag;
    int parity = a.parity;
    if (a.world > 1 && a.guard && tag == 0) {
        const int epoch = reinterpret_cast<const volatile int*>(a.guard)[MONO_GUARD_EPOCH];
        tag = (uint32_t)epoch * 256u + (uint32_t)a.site + 1u;
        parity = epoch & 1;
    }
    const uint64_t t0 = a.world > 1 ? globaltimer_ns() : 0;
    for (int idx = blockIdx.x * kReduceThreads + threadIdx.x; idx < total; idx += gridDim.x * kReduceThreads) {
        const int row = idx / pairs, pc = idx - row * pairs;
        float p0 = 0.f, p1 = 0.f;
#pragma unroll 4
        for (int s = 0; s < a.nsum; ++s) {
            const float2 v = *reinterpret_cast<const float2*>(a.partial + (size_t)s * a.sum_stride + (size_t)row * a.ld + 2 * pc);
            p0 += v.x;
            p1 += v.y;
        }
        float* out = a.out + (size_t)row * a.out_ld;
        if (a.world <= 1) {
            *reinterpret_cast<float2*>(out + 2 * pc) = make_float2(p0, p1);
            continue;
        }
        __nv_bfloat162 pb = __floats2bfloat162_rn(p0, p1);
        const uint32_t word = *reinterpret_cast<uint32_t*>(&pb);
        const size_t row_base = ((size_t)parity * kMaxRows + row) * all_pairs;
        const size_t my_off = (row_base + (size_t)a.rank * pairs + pc) * 8;
        for (int d = 0; d < a.world; ++d)
            if (d != a.rank) st_sys_v2(a.peer_ptrs[d] + my_off, word, tag);
        *reinterpret_cast<float2*>(out + (size_t)a.rank * a.n_local + 2 * pc) = make_float2(__low2float(pb), __high2float(pb));
        const uint64_t mine = a.peer_ptrs[a.rank];
        bool failed = guard_failed(a.guard);
        for (int src = 0; src < a.world && !failed; ++src) {
            if (src == a.rank) continue;
            const uint2 v = poll_tagged(mine + (row_base + (size_t)src * pairs + pc) * 8, tag, a.guard, a.peer_guards, a.world, a.rank,
                                        a.site, a.deadline_ns, t0, &failed);
            if (failed) break;
            const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&v.x);
            *reinterpret_cast<float2*>(out + (size_t)src * a.n_local + 2 * pc) = make_float2(__low2float(b), __high2float(b));
        }
    }
}

}  // namespace mono

// ------------------------------------------------------------------------ host
extern "C" int mono_act_prep_launch(const mono_act_prep_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->k < 128 || (a->k & 127) || a->k > 16384) {
        mono_set_error("mono_act_prep_launch: rows in 1..16 and k a multiple of 128 up to 16384 required");
        return MONO_E_ARG;
    }
    if ((a->src_bf16 == nullptr) == (a->src_f32 == nullptr)) {
        mono_set_error("mono_act_prep_launch: exactly one of src_bf16 / src_f32");
        return MONO_E_ARG;
    }
    if (a->planes) {
        const bool need_f32 = a->fmt == MONO_ACT_A8 || a->fmt == MONO_ACT_HILO;
        if ((need_f32 && !a->scale_f32) || ((a->fmt == MONO_ACT_MX8 || a->fmt == MONO_ACT_MX8N || a->fmt == MONO_ACT_NVF4) && !a->scale_e8) || a->fmt < 0 || a->fmt > MONO_ACT_NVF4) {
            mono_set_error("mono_act_prep_launch: format %d needs its scale buffer", a->fmt);
            return MONO_E_ARG;
        }
    }
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t ae = cudaFuncSetAttribute(mono::act_prep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 16384 * (int)sizeof(float));
        if (ae != cudaSuccess) {
            mono_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
            return (int)ae;
        }
        mono::attr_done(attr_once);
    }
    mono::launch_k(mono::act_prep_kernel, a->rows * (a->segs > 1 ? a->segs : 1), mono::kPrepThreads, a->k * sizeof(float), (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_act_prep_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_route_launch(const mono_route_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->n_experts < 1 || a->n_experts > mono::kMaxExperts ||
        a->top_k < 1 || a->top_k > 16 || a->top_k > a->n_experts || !a->logits || !a->ids || !a->weights ||
        !a->expert_list || !a->n_expert || !a->coef) {
        mono_set_error("mono_route_launch: rows 1..16, experts 1..512, top_k 1..16 and output pointers required");
        return MONO_E_ARG;
    }
    mono::launch_k(mono::route_kernel, 1, mono::kRouteThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_route_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

#ifdef MONO_TIMELINE
extern "C" int mono_timeline_read_rowdot(unsigned long long* out, int* ctas, int* points) {
    *ctas = MONO_TL_CTAS;
    *points = MONO_TL_POINTS;
    return (int)cudaMemcpyFromSymbol(out, mono::tl_rowdot, sizeof(unsigned long long) * MONO_TL_CTAS * MONO_TL_POINTS);
}
#endif

extern "C" int mono_rowdot_launch(const mono_rowdot_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->n < 1 || a->k < 128 || (a->k & 127) || !a->w || !a->x_bf16 || !a->out) {
        mono_set_error("mono_rowdot_launch: rows 1..16, k a multiple of 128 and all pointers required");
        return MONO_E_ARG;
    }
    // One wave of CTAs: a CTA holds a whole batch of loads in registers, so one CTA fits per SM; more columns
    // than SMs go two to a CTA (sharing the activation loads).  MONO_ROWDOT_COLS=1 / 2 forces the choice.
    const char* cf = getenv("MONO_ROWDOT_COLS");
    const int cols = cf ? (atoi(cf) == 2 ? 2 : 1) : (a->n > mono_sm_count() ? 2 : 1);
    // the rows staged in shared memory when they fit beside a resident CTA (8 rows x 7168: 112 KB): one round trip
    // for all activation loads instead of one per batch (MONO_ROWDOT_STAGED=0: read from global memory)
    const char* sf = getenv("MONO_ROWDOT_STAGED");
    const size_t xbytes = (size_t)a->rows * a->k * 2;
    const int staged = (!sf || sf[0] != '0') && xbytes <= 160 * 1024 && (reinterpret_cast<uintptr_t>(a->x_bf16) & 15) == 0 && (a->k & 7) == 0;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (staged && mono::attr_needed(attr_once)) {
        cudaError_t e1 = cudaFuncSetAttribute(mono::rowdot_kernel<1, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e1 == cudaSuccess) e1 = cudaFuncSetAttribute(mono::rowdot_kernel<2, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024);
        if (e1 != cudaSuccess) {
            mono_set_error("mono_rowdot_launch: %s", cudaGetErrorString(e1));
            return (int)e1;
        }
        mono::attr_done(attr_once);
    }
    if (cols == 2 && staged) mono::launch_k(mono::rowdot_kernel<2, true>, (a->n + 1) / 2, mono::kRowdotThreads, xbytes, (cudaStream_t)stream, *a);
    else if (cols == 2) mono::launch_k(mono::rowdot_kernel<2, false>, (a->n + 1) / 2, mono::kRowdotThreads, 0, (cudaStream_t)stream, *a);
    else if (staged) mono::launch_k(mono::rowdot_kernel<1, true>, a->n, mono::kRowdotThreads, xbytes, (cudaStream_t)stream, *a);
    else mono::launch_k(mono::rowdot_kernel<1, false>, a->n, mono::kRowdotThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_rowdot_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_router_launch(const mono_rowdot_args* d, const mono_route_args* r, int32_t* counter, void* stream) {
    if (!d || !r || !counter || d->rows < 1 || d->rows > MONO_MAX_ROWS || d->n < 1 || d->k < 128 || (d->k & 127) || !d->w ||
        !d->x_bf16 || !d->out) {
        mono_set_error("mono_router_launch: rows 1..16, k a multiple of 128, a counter and all pointers required");
        return MONO_E_ARG;
    }
    if (r->rows != d->rows || r->n_experts != d->n || r->n_experts > mono::kMaxExperts || r->top_k < 1 || r->top_k > 16 ||
        r->top_k > r->n_experts || r->logits != d->out || r->nsum != 1 || r->ld != d->out_ld || !r->ids || !r->weights ||
        !r->expert_list || !r->n_expert || !r->coef) {
        mono_set_error("mono_router_launch: the routing must read the logits this launch writes (same rows, experts and "
                       "leading dimension, one partial sum), experts 1..512, top_k 1..16");
        return MONO_E_ARG;
    }
    const int grid = (d->n + mono::kRouterCols - 1) / mono::kRouterCols;
    mono::launch_k(mono::router_kernel, grid, mono::kRouteThreads, 0, (cudaStream_t)stream, *d, *r, counter);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_router_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_mid_launch(const mono_mid_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->inter < 128 || (a->inter & 127) || !a->up || !a->planes ||
        a->max_slot < 1) {
        mono_set_error("mono_mid_launch: rows 1..16 and inter a multiple of 128 required");
        return MONO_E_ARG;
    }
    if ((a->fmt == MONO_ACT_A8 && !a->scale_f32) || ((a->fmt == MONO_ACT_MX8 || a->fmt == MONO_ACT_MX8N || a->fmt == MONO_ACT_NVF4) && !a->scale_e8) || a->fmt == MONO_ACT_HILO) {
        mono_set_error("mono_mid_launch: format %d not supported or missing scales", a->fmt);
        return MONO_E_ARG;
    }
    mono::launch_k(mono::mid_kernel, a->max_slot * a->rows, mono::kMidThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_mid_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

static int mid_check(const mono_mid_args* a) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->inter < 128 || (a->inter & 127) || !a->up || !a->planes || a->max_slot < 1) return 1;
    if ((a->fmt == MONO_ACT_A8 && !a->scale_f32) || ((a->fmt == MONO_ACT_MX8 || a->fmt == MONO_ACT_MX8N || a->fmt == MONO_ACT_NVF4) && !a->scale_e8) || a->fmt == MONO_ACT_HILO) return 1;
    return 0;
}

extern "C" int mono_mid_pair_launch(const mono_mid_args* a, const mono_mid_args* b, void* stream) {
    if (mid_check(a) || mid_check(b)) {
        mono_set_error("mono_mid_pair_launch: both stages need rows 1..16, inter a multiple of 128, buffers and a supported format");
        return MONO_E_ARG;
    }
    mono::launch_k(mono::mid_pair_kernel, a->max_slot * a->rows + b->max_slot * b->rows, mono::kMidThreads, 0, (cudaStream_t)stream, *a, *b);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_mid_pair_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" size_t mono_reduce_peer_bytes(int rows, int n, int world) {
    (void)rows;
    return (size_t)2 * world * MONO_MAX_ROWS * (n / 2) * 8;
}

static int reduce_args_check(const mono_reduce_args* a, const char* who) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->n < 2 || (a->n & 1) || !a->partial || !a->out || a->nsum < 1 || (a->ld & 1)) {
        mono_set_error("%s: rows 1..16, even n and ld, partial and out required", who);
        return MONO_E_ARG;
    }
    if (a->world > 1 && (!a->peer_ptrs || a->rank < 0 || a->rank >= a->world || a->world > 8 || a->deadline_ns == 0 ||
                         (a->tag == 0 && !a->guard) || a->site < 0 || a->site > 254)) {
        mono_set_error("%s: world %d needs peer_ptrs, a rank, a deadline, a site in 0..254 and a tag or guard words", who, a->world);
        return MONO_E_ARG;
    }
    if (a->rsag && (a->world < 2 || (a->n / 2) % (2 * a->world) != 0)) {
        mono_set_error("%s: the reduce-scatter form needs world > 1 and n / 2 = %d divisible by 2 x world = %d", who, a->n / 2, 2 * a->world);
        return MONO_E_ARG;
    }
    return 0;
}

extern "C" int mono_reduce_launch(const mono_reduce_args* a, void* stream) {
    if (int rc = reduce_args_check(a, "mono_reduce_launch")) return rc;
    const int total = a->rows * (a->n / 2);
    int grid = (total + mono::kReduceThreads - 1) / mono::kReduceThreads;
    const int sms = mono_sm_count();
    if (grid > 2 * sms) grid = 2 * sms;
    mono::launch_k(mono::reduce_kernel, grid, mono::kReduceThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_reduce_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_reduce_norm_launch(const mono_reduce_args* r, const mono_act_prep_args* a, void* stream) {
    if (int rc = reduce_args_check(r, "mono_reduce_norm_launch")) return rc;
    if (!a || a->rows != r->rows || a->k != r->n || a->k < 128 || (a->k & 127) || a->k > 16384 || a->segs > 1 || (r->ld & 3) ||
        (reinterpret_cast<uintptr_t>(r->partial) & 15) || (reinterpret_cast<uintptr_t>(r->out) & 7) ||
        (r->residual && (reinterpret_cast<uintptr_t>(r->residual) & 7))) {
        mono_set_error("mono_reduce_norm_launch: the staging must take the reduction's rows (same rows, k = n a multiple of 128 up to "
                       "16384, no segments, ld a multiple of 4, 16-byte aligned partial sums)");
        return MONO_E_ARG;
    }
    if (a->planes) {
        const bool need_f32 = a->fmt == MONO_ACT_A8 || a->fmt == MONO_ACT_HILO;
        if ((need_f32 && !a->scale_f32) || ((a->fmt == MONO_ACT_MX8 || a->fmt == MONO_ACT_MX8N || a->fmt == MONO_ACT_NVF4) && !a->scale_e8) || a->fmt < 0 || a->fmt > MONO_ACT_NVF4) {
            mono_set_error("mono_reduce_norm_launch: format %d needs its scale buffer", a->fmt);
            return MONO_E_ARG;
        }
    }
    // the largest cluster (8, 4, 2, 1 CTAs per row) whose CTAs get whole 128-column chunks, at most 2048 columns each
    int c = 8;
    while (c > 1 && (a->k % (c * 128)) != 0) c >>= 1;
    if (a->k / c > 2048) {
        mono_set_error("mono_reduce_norm_launch: k = %d leaves more than 2048 columns per CTA of the row's cluster", a->k);
        return MONO_E_ARG;
    }
    const size_t smem = (size_t)(a->k / c) * sizeof(float);
    const cudaStream_t st = (cudaStream_t)stream;
    if (c == 8) mono::launch_k(mono::reduce_norm_kernel<8>, r->rows * 8, mono::kRnThreads, smem, st, *r, *a);
    else if (c == 4) mono::launch_k(mono::reduce_norm_kernel<4>, r->rows * 4, mono::kRnThreads, smem, st, *r, *a);
    else if (c == 2) mono::launch_k(mono::reduce_norm_kernel<2>, r->rows * 2, mono::kRnThreads, smem, st, *r, *a);
    else mono::launch_k(mono::reduce_norm_kernel<1>, r->rows, mono::kRnThreads, smem, st, *r, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_reduce_norm_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_l2_prefetch_launch(const mono_prefetch_args* a, void* stream) {
    if (!a || a->n < 1 || a->n > MONO_PREFETCH_RANGES) {
        mono_set_error("mono_l2_prefetch_launch: 1..%d ranges required", MONO_PREFETCH_RANGES);
        return MONO_E_ARG;
    }
    for (int r = 0; r < a->n; ++r)
        if (!a->ptr[r] || (a->ptr[r] & 15) || a->bytes[r] < 16) {
            mono_set_error("mono_l2_prefetch_launch: range %d needs a 16-byte aligned address and at least 16 bytes", r);
            return MONO_E_ARG;
        }
    mono::launch_k(mono::l2_prefetch_kernel, mono_sm_count(), 128, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_l2_prefetch_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_epoch_advance_launch(int32_t* guard, void* stream) {
    if (!guard) return MONO_E_ARG;
    mono::launch_k(mono::epoch_advance_kernel, 1, 1, 0, (cudaStream_t)stream, guard);
    return (int)cudaGetLastError();
}

extern "C" size_t mono_logits_peer_bytes(int n_local, int world) {
    return (size_t)2 * MONO_MAX_ROWS * ((size_t)world * n_local / 2) * 8;
}

extern "C" int mono_logits_gather_launch(const mono_logits_gather_args* a, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->n_local < 2 || (a->n_local & 1) || (a->ld & 1) || !a->partial || !a->out ||
        a->nsum < 1 || a->world < 1 || a->out_ld < a->world * a->n_local || (a->out_ld & 1)) {
        mono_set_error("mono_logits_gather_launch: rows 1..16, even n_local and ld, partial, out and out_ld >= world * n_local required");
        return MONO_E_ARG;
    }
    if (a->world > 1 && (!a->peer_ptrs || a->rank < 0 || a->rank >= a->world || a->world > 8 || a->deadline_ns == 0 ||
                         (a->tag == 0 && !a->guard) || a->site < 0 || a->site > 254)) {
        mono_set_error("mono_logits_gather_launch: world %d needs peer_ptrs, a rank, a deadline, a site in 0..254 and a tag or guard words",
                       a->world);
        return MONO_E_ARG;
    }
    const int total = a->rows * (a->n_local / 2);
    int grid = (total + mono::kReduceThreads - 1) / mono::kReduceThreads;
    const int sms = mono_sm_count();
    if (grid > 8 * sms) grid = 8 * sms;
    mono::launch_k(mono::logits_gather_kernel, grid, mono::kReduceThreads, 0, (cudaStream_t)stream, *a);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_logits_gather_launch: %s", cudaGetErrorString(e));
    return (int)e;
}
