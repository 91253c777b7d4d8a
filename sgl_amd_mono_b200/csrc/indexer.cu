// Lightning indexer: scores of every causal key and the exact top-k of each row.
//
// Reference counterparts: glm53/gfx950/kernel.py:2684-3000 (index score: sum over
// heads of relu(q_h . k) * w_h in f32), :2698-2699 (radix key), :3002-3636 (exact
// top-k: histogram passes, candidates, ties to the lowest position, ordered gather)
// and :3341-3346 (publication as global KV slots); FP4 index keys with one E8M0 code
// per 32 dims as deepseek_v4/gfx950/kernels/stages/indexer.py:143-151.
#include <cstdlib>
#include <cooperative_groups.h>
#include "mono_common.cuh"

namespace cg = cooperative_groups;

extern void mono_set_error(const char* fmt, ...);

namespace mono {

// ------------------------------------------------------------------ scores
constexpr int kScoreThreads = 256;
constexpr int kKeyTile = 128;
constexpr int kTilesPerTask = 2;
constexpr int kIdxPitch = 128 + 8;  // bf16 elements per staged row (272 B: conflict-free ldmatrix)

struct ScoreSmem {
    __nv_bfloat16 keys[kKeyTile][kIdxPitch];
    __nv_bfloat16 q[64][kIdxPitch];
    float w[64];
};

__global__ void __launch_bounds__(kScoreThreads) index_score_kernel(const mono_index_args a, int max_tiles) {
    pdl_prologue();
    extern __shared__ uint8_t smem_raw[];
    ScoreSmem& sm = *reinterpret_cast<ScoreSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const int mtiles = (a.index_heads + 15) >> 4;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.idx_q);
    // a task = kTilesPerTask consecutive key tiles of one row: the row's queries and head weights are staged once
    const int groups = (max_tiles + kTilesPerTask - 1) / kTilesPerTask;
    for (int task = blockIdx.x; task < a.rows * groups; task += gridDim.x) {
        const int row = task / groups, tile0 = (task - row * groups) * kTilesPerTask;
        if (a.slots && a.slots[row] < 0) continue;
        const int n = (int)a.positions[row] + 1;
        if (tile0 * kKeyTile >= n) continue;
        __syncthreads();
        // ---- stage q (zero rows past index_heads) and the head weights
        for (int c = tid; c < 64 * 16; c += kScoreThreads) {
            const int h = c >> 4, ch = c & 15;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (h < a.index_heads) v = *reinterpret_cast<const uint4*>(qg + ((size_t)row * a.index_heads + h) * 128 + ch * 8);
            *reinterpret_cast<uint4*>(&sm.q[h][ch * 8]) = v;
        }
        if (tid < 64) sm.w[tid] = tid < a.index_heads ? a.idx_w[(size_t)row * a.w_ld + tid] : 0.f;
        for (int tile = tile0; tile < tile0 + kTilesPerTask && tile * kKeyTile < n; ++tile) {
        if (tile != tile0) __syncthreads();  // every warp is done with the previous tile's keys
        // ---- stage 128 keys: E2M1 * 2^(code - 127) is exact in bf16
        {
            const int key = tid >> 1, half = tid & 1;
            const int p = tile * kKeyTile + key;
            uint4 v0 = make_uint4(0, 0, 0, 0), v1 = v0;
            uint32_t codes = 0x7f7f;
            if (p < n) {
                const int64_t pg = a.page_table[(size_t)row * a.pt_ld + p / kPage];
                if (pg >= 0 && pg < a.n_pages) {
                    const uint8_t* page = a.idx_pages + (size_t)pg * kIdxPageBytes;
                    const int off = p % kPage;
                    const uint4* src = reinterpret_cast<const uint4*>(page + (size_t)off * 64 + half * 32);
                    v0 = __ldg(src);
                    v1 = __ldg(src + 1);
                    codes = __ldg(reinterpret_cast<const uint16_t*>(page + kPage * 64 + off * 4 + half * 2));
                }
            }
            const uint32_t words[8] = {v0.x, v0.y, v0.z, v0.w, v1.x, v1.y, v1.z, v1.w};
            __nv_bfloat16* dst = &sm.keys[key][half * 64];
#pragma unroll
            for (int wi = 0; wi < 8; ++wi) {
                // an E2M1 code moved to the top of an f16's exponent/mantissa reads as value * 2^-14
                // (subnormal 0.5 included), so the block scale carries the 2^14
                const float sc = exp2_code(max((int)((codes >> ((wi >> 2) * 8)) & 0xFF), 1)) * 16384.f;
                uint32_t o[4];
#pragma unroll
                for (int b = 0; b < 4; ++b) {
                    const uint32_t byte = (words[wi] >> (8 * b)) & 0xFF;
                    const uint32_t h2 = ((byte & 7u) << 9) | ((byte & 8u) << 12) | ((byte & 0x70u) << 21) | ((byte & 0x80u) << 24);
                    const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&h2));
                    __nv_bfloat162 pr = __floats2bfloat162_rn(f.x * sc, f.y * sc);
                    o[b] = *reinterpret_cast<uint32_t*>(&pr);
                }
                *reinterpret_cast<uint4*>(dst + wi * 8) = make_uint4(o[0], o[1], o[2], o[3]);
            }
        }
        __syncthreads();
        // ---- dots[head][key] on bf16 MMAs: warp w owns keys 16w .. 16w+15
        float acc[4][2][4];
#pragma unroll
        for (int m = 0; m < 4; ++m)
#pragma unroll
            for (int nn = 0; nn < 2; ++nn)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[m][nn][i] = 0.f;
#pragma unroll
        for (int ks = 0; ks < 8; ++ks) {
            uint32_t bfr[2][2];
#pragma unroll
            for (int nn = 0; nn < 2; ++nn)
                ldmatrix_x2(bfr[nn], smem_u32(&sm.keys[warp * 16 + nn * 8 + (lane & 7)][((lane >> 3) & 1) * 8]) + ks * 32);
#pragma unroll
            for (int m = 0; m < 4; ++m) {
                if (m < mtiles) {
                    uint32_t af[4];
                    ldmatrix_x4(af, smem_u32(&sm.q[m * 16 + (lane & 15)][(lane >> 4) * 8]) + ks * 32);
#pragma unroll
                    for (int nn = 0; nn < 2; ++nn) mma_bf16(acc[m][nn], af[0], af[1], af[2], af[3], bfr[nn][0], bfr[nn][1]);
                }
            }
        }
        // ---- score[key] = sum_h relu(dot) * w_h
#pragma unroll
        for (int nn = 0; nn < 2; ++nn) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                float s = 0.f;
#pragma unroll
                for (int m = 0; m < 4; ++m) {
                    if (m < mtiles) {
                        s += fmaxf(acc[m][nn][c], 0.f) * sm.w[m * 16 + g];
                        s += fmaxf(acc[m][nn][2 + c], 0.f) * sm.w[m * 16 + g + 8];
                    }
                }
                s += __shfl_xor_sync(0xffffffffu, s, 4);
                s += __shfl_xor_sync(0xffffffffu, s, 8);
                s += __shfl_xor_sync(0xffffffffu, s, 16);
                const int p = tile * kKeyTile + warp * 16 + nn * 8 + 2 * t4 + c;
                if (g == 0 && p < n) a.scores[(size_t)row * a.score_ld + p] = s;
            }
        }
        }  // tiles of the task
    }
}

// ------------------------------------------------------------------ exact top-k
// One CTA per row.  Four 8-bit radix passes find the k-th largest key exactly; one
// ordered pass gathers [keys above it in position order] ++ [first ties in position order].
constexpr int kTopkThreads = 1024;

__device__ __forceinline__ uint32_t score_key(float f) {
    const uint32_t b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b ^ 0x80000000u);
}

__global__ void __launch_bounds__(kTopkThreads, 1) index_topk_kernel(const mono_index_args a, int smem_keys) {
    pdl_prologue();
    extern __shared__ uint32_t skeys[];  // the row's radix keys when they fit (smem_keys != 0)
    __shared__ int hist[256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_krem;
    __shared__ int wsum_gt[kTopkThreads / 32], wsum_eq[kTopkThreads / 32];
    const int row = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int32_t* out = a.topk_slots + (size_t)row * a.topk;
    int32_t* outp = a.topk_pos ? a.topk_pos + (size_t)row * a.topk : nullptr;
    const bool live = !a.slots || a.slots[row] >= 0;
    const int n = live ? (int)a.positions[row] + 1 : 0;
    const int32_t* pt = a.page_table + (size_t)row * a.pt_ld;
    if (n <= a.topk) {
        for (int i = tid; i < a.topk; i += kTopkThreads) {
            int32_t v = -1;
            if (i < n) v = pt[i / kPage] * kPage + i % kPage;
            out[i] = v;
            if (outp) outp[i] = i < n ? i : -1;
        }
        return;
    }
    const float* sc = a.scores + (size_t)row * a.score_ld;
    if (smem_keys) {
        // one pass over global memory with every load in flight; the radix passes then run on-chip
#pragma unroll 8
        for (int i = tid; i < n; i += kTopkThreads) skeys[i] = score_key(sc[i]);
    }
    if (tid == 0) { s_prefix = 0; s_krem = a.topk; }
    for (int pass = 3; pass >= 0; --pass) {
        if (tid < 256) hist[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const int krem = s_krem;
        const int shift = pass * 8;
        // scores of one row share their leading bytes, so most keys of a pass fall into a
        // few bins: lanes that hit the same bin are counted by one atomic (match + popc)
        // (a thread counts runs of equal bins itself and adds each run with one atomic)
        int cur = -1, run = 0;
        for (int i = tid; i < n; i += kTopkThreads) {
            const uint32_t k = smem_keys ? skeys[i] : score_key(sc[i]);
            if (pass == 3 || (k >> (shift + 8)) == prefix) {
                const int bin = (int)((k >> shift) & 0xFF);
                if (bin == cur) {
                    ++run;
                } else {
                    if (run) atomicAdd(&hist[cur], run);
                    cur = bin;
                    run = 1;
                }
            }
        }
        {
            const int c0 = __shfl_sync(0xffffffffu, cur, 0);
            if (__all_sync(0xffffffffu, cur == c0 && run > 0)) {  // the whole warp ends in one bin
                const int tot = __reduce_add_sync(0xffffffffu, run);
                if (lane == 0) atomicAdd(&hist[c0], tot);
            } else if (run) {
                atomicAdd(&hist[cur], run);
            }
        }
        __syncthreads();
        // keys above digit d = suffix sum of the histogram: a warp scan plus 8 warp totals
        int mine = 0, suffix = 0;
        if (tid < 256) {
            mine = hist[tid];
            suffix = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, suffix, o);
                if (lane + o < 32) suffix += t;
            }
            if (lane == 0) wsum_gt[warp] = suffix;  // total of digits 32 * warp .. 32 * warp + 31
        }
        __syncthreads();
        if (tid < 256) {
            int above = suffix - mine;
            for (int w = warp + 1; w < 8; ++w) above += wsum_gt[w];
            if (above < krem && krem <= above + mine) {
                s_prefix = (prefix << 8) | (uint32_t)tid;
                s_krem = krem - above;
            }
        }
        __syncthreads();
    }
    const uint32_t thr = s_prefix;
    const int remain = s_krem;  // ties to take
    const int n_gt = a.topk - remain;
    // ordered gather: a warp owns a contiguous range of positions and walks it 32 at a time
    // (consecutive lanes read consecutive keys); ballots give the order inside a group
    const int seg = (((n + 31) / 32 + 31) / 32) * 32;  // positions per warp, a multiple of 32
    const int lo = min(warp * seg, n), hi = min(lo + seg, n);
    const uint32_t lt = (1u << lane) - 1;
    int c_gt = 0, c_eq = 0;  // warp totals (the same in every lane)
    for (int i0 = lo; i0 < hi; i0 += 32) {
        const int i = i0 + lane;
        const uint32_t k = i < hi ? (smem_keys ? skeys[i] : score_key(sc[i])) : 0u;
        c_gt += __popc(__ballot_sync(0xffffffffu, i < hi && k > thr));
        c_eq += __popc(__ballot_sync(0xffffffffu, i < hi && k == thr));
    }
    if (lane == 0) { wsum_gt[warp] = c_gt; wsum_eq[warp] = c_eq; }
    __syncthreads();
    int o_gt = 0, o_eq = 0;  // exclusive prefixes over the warps before this one
    {
        const int g0 = lane < warp ? wsum_gt[lane] : 0, e0 = lane < warp ? wsum_eq[lane] : 0;
        o_gt = __reduce_add_sync(0xffffffffu, g0);
        o_eq = __reduce_add_sync(0xffffffffu, e0);
    }
    for (int i0 = lo; i0 < hi; i0 += 32) {
        const int i = i0 + lane;
        const uint32_t k = i < hi ? (smem_keys ? skeys[i] : score_key(sc[i])) : 0u;
        const bool gt = i < hi && k > thr, eq = i < hi && k == thr;
        const uint32_t m_gt = __ballot_sync(0xffffffffu, gt), m_eq = __ballot_sync(0xffffffffu, eq);
        int dst = -1;
        if (gt) dst = o_gt + __popc(m_gt & lt);
        else if (eq) { const int e = o_eq + __popc(m_eq & lt); if (e < remain) dst = n_gt + e; }
        if (dst >= 0) {
            out[dst] = pt[i / kPage] * kPage + i % kPage;
            if (outp) outp[dst] = i;
        }
        o_gt += __popc(m_gt);
        o_eq += __popc(m_eq);
    }
}

// The same selection for rows of up to 16K positions by a cluster of eight CTAs per row: CTA c of
// the cluster holds positions 2048 c .. 2048 c + 2047 in registers (two keys per thread).  A pass
// counts into the CTA's own histogram; after one cluster barrier every CTA adds the eight histograms
// over distributed shared memory and takes the same decision.  The histograms alternate between two
// buffers, so a pass needs one cluster barrier: a buffer is zeroed again only after the barrier of
// the pass in between, which no CTA reaches before it has read that buffer.  Output order as above.
constexpr int kClSize = 8;
constexpr int kClKeys = 2;
constexpr int kClSpan = kTopkThreads * kClKeys;

__global__ void __cluster_dims__(kClSize, 1, 1) __launch_bounds__(kTopkThreads, 1)
    index_topk_cluster_kernel(const mono_index_args a) {
    pdl_launch_dependents();
    if (threadIdx.x == 0) {  // during the wait for the scores: the step's tables of this row
        prefetch_l2(a.positions + blockIdx.x / kClSize);
        prefetch_l2(a.page_table + (size_t)(blockIdx.x / kClSize) * a.pt_ld);
    }
    pdl_wait();
    cg::cluster_group cluster = cg::this_cluster();
    __shared__ int hist[2][256];
    __shared__ uint32_t s_prefix;
    __shared__ int s_krem;
    __shared__ int wsum[8];
    __shared__ int cnt_gt[kClKeys * 32], cnt_eq[kClKeys * 32];  // [j][warp], then their exclusive prefixes
    __shared__ int part_gt[kClKeys], part_eq[kClKeys];
    __shared__ int ctot[2];    // this CTA's keys above the threshold / equal to it
    __shared__ int s_base[2];  // the same, summed over the CTAs before this one
    const int row = blockIdx.x / kClSize, crank = (int)cluster.block_rank();
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    int32_t* out = a.topk_slots + (size_t)row * a.topk;
    int32_t* outp = a.topk_pos ? a.topk_pos + (size_t)row * a.topk : nullptr;
    const bool live = !a.slots || a.slots[row] >= 0;
    const int n = live ? (int)a.positions[row] + 1 : 0;
    const int32_t* pt = a.page_table + (size_t)row * a.pt_ld;
    if (n <= a.topk) {  // the same for every CTA of the cluster: none of them reaches a cluster barrier
        if (crank == 0) {
            for (int i = tid; i < a.topk; i += kTopkThreads) {
                int32_t v = -1;
                if (i < n) v = pt[i / kPage] * kPage + i % kPage;
                out[i] = v;
                if (outp) outp[i] = i < n ? i : -1;
            }
        }
        return;
    }
    const float* sc = a.scores + (size_t)row * a.score_ld;
    const int pos0 = crank * kClSpan + tid;
    uint32_t key[kClKeys];
#pragma unroll
    for (int j = 0; j < kClKeys; ++j) {
        const int i = pos0 + j * kTopkThreads;
        key[j] = i < n ? score_key(sc[i]) : 0u;
    }
    if (tid == 0) { s_prefix = 0; s_krem = a.topk; }
    for (int pass = 3; pass >= 0; --pass) {
        int* h = hist[pass & 1];
        if (tid < 256) h[tid] = 0;
        __syncthreads();
        const uint32_t prefix = s_prefix;
        const int krem = s_krem;
        const int shift = pass * 8;
        int cur = -1, run = 0;
#pragma unroll
        for (int j = 0; j < kClKeys; ++j) {
            const uint32_t k = key[j];
            if (pos0 + j * kTopkThreads < n && (pass == 3 || (k >> (shift + 8)) == prefix)) {
                const int bin = (int)((k >> shift) & 0xFF);
                if (bin == cur) {
                    ++run;
                } else {
                    if (run) atomicAdd(&h[cur], run);
                    cur = bin;
                    run = 1;
                }
            }
        }
        {
            const int c0 = __shfl_sync(0xffffffffu, cur, 0);
            if (__all_sync(0xffffffffu, cur == c0 && run > 0)) {  // the whole warp ends in one bin
                const int tot = __reduce_add_sync(0xffffffffu, run);
                if (lane == 0) atomicAdd(&h[c0], tot);
            } else if (run) {
                atomicAdd(&h[cur], run);
            }
        }
        cluster.sync();
        int mine = 0, suffix = 0;
        if (tid < 256) {
#pragma unroll
            for (int r = 0; r < kClSize; ++r) mine += cluster.map_shared_rank(h, r)[tid];
            suffix = mine;
#pragma unroll
            for (int o = 1; o < 32; o <<= 1) {
                const int t = __shfl_down_sync(0xffffffffu, suffix, o);
                if (lane + o < 32) suffix += t;
            }
            if (lane == 0) wsum[warp] = suffix;
        }
        __syncthreads();
        if (tid < 256) {
            int above = suffix - mine;
            for (int w = warp + 1; w < 8; ++w) above += wsum[w];
            if (above < krem && krem <= above + mine) {
                s_prefix = (prefix << 8) | (uint32_t)tid;
                s_krem = krem - above;
            }
        }
        __syncthreads();
    }
    const uint32_t thr = s_prefix;
    const int remain = s_krem;  // ties to take
    const int n_gt = a.topk - remain;
    // position order = (CTA, j, warp, lane)
    const uint32_t lt = (1u << lane) - 1;
#pragma unroll
    for (int j = 0; j < kClKeys; ++j) {
        const bool ok = pos0 + j * kTopkThreads < n;
        const uint32_t m_gt = __ballot_sync(0xffffffffu, ok && key[j] > thr);
        const uint32_t m_eq = __ballot_sync(0xffffffffu, ok && key[j] == thr);
        if (lane == 0) { cnt_gt[j * 32 + warp] = __popc(m_gt); cnt_eq[j * 32 + warp] = __popc(m_eq); }
    }
    __syncthreads();
    int g = 0, e = 0, gi = 0, ei = 0;
    if (tid < kClKeys * 32) {
        g = gi = cnt_gt[tid];
        e = ei = cnt_eq[tid];
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int tg = __shfl_up_sync(0xffffffffu, gi, o), te = __shfl_up_sync(0xffffffffu, ei, o);
            if (lane >= o) { gi += tg; ei += te; }
        }
        if (lane == 31) { part_gt[warp] = gi; part_eq[warp] = ei; }
    }
    __syncthreads();
    if (tid < kClKeys * 32) {
        int bg = 0, be = 0;
        for (int w = 0; w < warp; ++w) { bg += part_gt[w]; be += part_eq[w]; }
        cnt_gt[tid] = bg + gi - g;
        cnt_eq[tid] = be + ei - e;
    }
    if (tid == 0) {
        int tg = 0, te = 0;
        for (int w = 0; w < kClKeys; ++w) { tg += part_gt[w]; te += part_eq[w]; }
        ctot[0] = tg;
        ctot[1] = te;
    }
    cluster.sync();
    if (warp == 0) {
        int bg = 0, be = 0;
        if (lane < crank) {
            const int* rt = cluster.map_shared_rank(ctot, lane);
            bg = rt[0];
            be = rt[1];
        }
        bg = __reduce_add_sync(0xffffffffu, bg);
        be = __reduce_add_sync(0xffffffffu, be);
        if (lane == 0) { s_base[0] = bg; s_base[1] = be; }
    }
    __syncthreads();
    const int base_gt = s_base[0], base_eq = s_base[1];
#pragma unroll
    for (int j = 0; j < kClKeys; ++j) {
        const int i = pos0 + j * kTopkThreads;
        const bool ok = i < n;
        const bool gt = ok && key[j] > thr, eq = ok && key[j] == thr;
        const uint32_t m_gt = __ballot_sync(0xffffffffu, gt), m_eq = __ballot_sync(0xffffffffu, eq);
        int dst = -1;
        if (gt) dst = base_gt + cnt_gt[j * 32 + warp] + __popc(m_gt & lt);
        else if (eq) { const int q = base_eq + cnt_eq[j * 32 + warp] + __popc(m_eq & lt); if (q < remain) dst = n_gt + q; }
        if (dst >= 0) {
            out[dst] = pt[i / kPage] * kPage + i % kPage;
            if (outp) outp[dst] = i;
        }
    }
    cluster.sync();  // no CTA leaves while another may still read its shared memory
}

}  // namespace mono

int mono_index_score_tc_launch(const mono_index_args* a, void* stream);  // index_score_tc.cu

static int check_index_args(const mono_index_args* a, const char* who) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->index_heads < 1 || a->index_heads > 64 || a->topk < 1 ||
        !a->page_table || !a->positions || !a->scores || a->score_ld < 1) {
        mono_set_error("%s: rows 1..16, index_heads 1..64, topk >= 1 and the step tables required", who);
        return MONO_E_ARG;
    }
    return 0;
}

extern "C" int mono_index_score_launch(const mono_index_args* a, void* stream) {
    if (int rc = check_index_args(a, "mono_index_score_launch")) return rc;
    if ((!a->idx_q && !a->iq) || !a->idx_w || !a->idx_pages) {
        mono_set_error("mono_index_score_launch: idx_q (or iq), idx_w and idx_pages required");
        return MONO_E_ARG;
    }
    if (a->iq && (!a->cos || !a->sin || a->iq_nsum < 1 || (a->iq_ld & 3) || (a->iq_sum_stride & 3) ||
                  (reinterpret_cast<uintptr_t>(a->iq) & 15) || (reinterpret_cast<uintptr_t>(a->idx_q) & 7))) {
        mono_set_error("mono_index_score_launch: iq needs cos, sin, iq_nsum >= 1 and 16-byte aligned rows");
        return MONO_E_ARG;
    }
    {
        // the tcgen05 kernel (MONO_INDEX_SCORE_TC=0: the mma.sync kernel below)
        const char* sw = getenv("MONO_INDEX_SCORE_TC");
        if ((!sw || sw[0] != '0') && !(reinterpret_cast<uintptr_t>(a->idx_pages) & 15) && !(reinterpret_cast<uintptr_t>(a->idx_q) & 15)) {
            const int rc = mono_index_score_tc_launch(a, stream);
            if (rc != 0) mono_set_error("mono_index_score_launch: %s", cudaGetErrorString((cudaError_t)rc));
            return rc;
        }
    }
    if (a->iq) {
        mono_set_error("mono_index_score_launch: index queries from partial sums (iq) are made by the tcgen05 kernel only");
        return MONO_E_ARG;
    }
    const size_t smem = sizeof(mono::ScoreSmem) + 128;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t ae = cudaFuncSetAttribute(mono::index_score_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (ae != cudaSuccess) {
            mono_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
            return (int)ae;
        }
        mono::attr_done(attr_once);
    }
    const int max_tiles = (a->score_ld + mono::kKeyTile - 1) / mono::kKeyTile;
    int grid = a->rows * ((max_tiles + mono::kTilesPerTask - 1) / mono::kTilesPerTask);
    const int sms = mono_sm_count();
    if (grid > 4 * sms) grid = 4 * sms;
    mono::launch_k(mono::index_score_kernel, grid, mono::kScoreThreads, smem, (cudaStream_t)stream, *a, max_tiles);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_index_score_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" int mono_index_topk_launch(const mono_index_args* a, void* stream) {
    if (int rc = check_index_args(a, "mono_index_topk_launch")) return rc;
    if (!a->topk_slots) {
        mono_set_error("mono_index_topk_launch: topk_slots required");
        return MONO_E_ARG;
    }
    // rows of up to 16K positions: a cluster of eight CTAs per row (MONO_TOPK_CLUSTER=0: the general kernel)
    if (a->score_ld <= mono::kClSize * mono::kClSpan) {
        const char* sw = getenv("MONO_TOPK_CLUSTER");
        if (!sw || sw[0] != '0') {
            mono::launch_k(mono::index_topk_cluster_kernel, a->rows * mono::kClSize, mono::kTopkThreads, 0, (cudaStream_t)stream, *a);
            cudaError_t e = cudaGetLastError();
            if (e != cudaSuccess) mono_set_error("mono_index_topk_launch: %s", cudaGetErrorString(e));
            return (int)e;
        }
    }
    // rows of up to 48K keys keep their radix keys in shared memory
    const size_t key_bytes = (size_t)a->score_ld * sizeof(uint32_t);
    const int smem_keys = key_bytes <= 192 * 1024 ? 1 : 0;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        const cudaError_t ae = cudaFuncSetAttribute(mono::index_topk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 192 * 1024);
        if (ae != cudaSuccess) {
            mono_set_error("cudaFuncSetAttribute: %s", cudaGetErrorString(ae));
            return (int)ae;
        }
        mono::attr_done(attr_once);
    }
    mono::launch_k(mono::index_topk_kernel, a->rows, mono::kTopkThreads, smem_keys ? key_bytes : 0, (cudaStream_t)stream, *a, smem_keys);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_index_topk_launch: %s", cudaGetErrorString(e));
    return (int)e;
}
