// Sparse MLA decode attention over the selected KV slots (the operator of BASELINE
// config 2, and the attention stage of the layer).
//
// Reference counterpart: glm53/gfx950/kernel.py:3638-3973 (split: 64 keys per task,
// split-local max / sum, p rounded to bf16 before P.V, bf16 partial accumulator) and
// :3975-4075 (merge: w_j = e^(m_j - M) / sum_j l_j e^(m_j - M)).
//
// sm_100a design: a task is (row, group of 16 heads, run of 64-key chunks).  The CTA gathers
// each chunk's 64 cache rows (576 E4M3 bytes + one f32 scale each) with 16-byte loads that are
// all in flight at once, widens them to bf16 in shared memory, and runs Q.K^T and P.V on bf16
// warp MMAs with the running maximum / sum and the output accumulators in registers, so a task
// writes one partial however many chunks it covers (the reference writes one per 64 keys).
#include <cstdlib>
#include "mono_common.cuh"
#include "act_quant.cuh"

extern void mono_set_error(const char* fmt, ...);

namespace mono {

constexpr int kSplit = 64;             // keys per task
constexpr int kKvPitch = kKvDim + 8;   // bf16 elements per staged key row (1168 B: conflict-free ldmatrix)
constexpr int kPPitch = kSplit + 8;
constexpr int kMlaThreads = 256;
constexpr int kHeadGroup = 16;

struct MlaSmem {
    __nv_bfloat16 kv[kSplit][kKvPitch];
    __nv_bfloat16 q[kHeadGroup][kKvPitch];
    __nv_bfloat16 p[kHeadGroup][kPPitch];
    float s[kHeadGroup][kSplit];
    float ml[kHeadGroup][2];
    int valid[kSplit];
};

__device__ __forceinline__ void e4m3x16_to_bf16(const uint4& v, float scale, __nv_bfloat16* dst) {
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
    uint32_t o[8];
#pragma unroll
    for (int i = 0; i < 4; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const __nv_fp8x2_storage_t pr = (__nv_fp8x2_storage_t)((w[i] >> (16 * h)) & 0xFFFF);
            const __half2_raw hr = __nv_cvt_fp8x2_to_halfraw2(pr, __NV_E4M3);
            const float2 f = __half22float2(*reinterpret_cast<const __half2*>(&hr));
            __nv_bfloat162 b = __floats2bfloat162_rn(f.x * scale, f.y * scale);
            o[2 * i + h] = *reinterpret_cast<uint32_t*>(&b);
        }
    }
    // consecutive lanes write consecutive 32-byte pieces: lanes 4..7 of every eight store their halves in the
    // other order, so that eight lanes' 16-byte stores fall into eight different bank groups
    const int swap = (threadIdx.x >> 2) & 1;
    const uint4 lo = make_uint4(o[0], o[1], o[2], o[3]), hi = make_uint4(o[4], o[5], o[6], o[7]);
    *reinterpret_cast<uint4*>(dst + 8 * swap) = swap ? hi : lo;
    *reinterpret_cast<uint4*>(dst + 8 * (1 - swap)) = swap ? lo : hi;
}

// A task is (row, head group of 16, run of `chunks` 64-key chunks).  The 16 heads' queries are staged
// once; every chunk is gathered, widened, scored, and folded into accumulators that stay in registers
// (running maximum and sum per head, rescaled like a flash-decoding pass), so a task writes one partial
// however many chunks it covers.  Two CTAs per SM overlap one's gather with the other's MMAs.
__global__ void __launch_bounds__(kMlaThreads, 2) sparse_mla_split_kernel(const mono_sparse_mla_args a, int nsplit, int chunks) {
    pdl_prologue();
    extern __shared__ uint8_t smem_raw[];
    MlaSmem& sm = *reinterpret_cast<MlaSmem*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    __shared__ float s_scale[kHeadGroup];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t4 = lane & 3;
    const __nv_bfloat16* qg = reinterpret_cast<const __nv_bfloat16*>(a.q);
    __nv_bfloat16* part_acc = reinterpret_cast<__nv_bfloat16*>(a.scratch);
    float* part_ml = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(a.scratch) +
                                              (size_t)a.rows * nsplit * a.heads * 512 * sizeof(__nv_bfloat16));
    const int hgroups = (a.heads + kHeadGroup - 1) / kHeadGroup;
    const int total_chunks = (a.topk + kSplit - 1) / kSplit;

    for (int task = blockIdx.x; task < a.rows * hgroups * nsplit; task += gridDim.x) {
        const int sp = task % nsplit, hg = (task / nsplit) % hgroups, row = task / (nsplit * hgroups);
        __syncthreads();
        // ---- stage the 16 heads of q, reset the running statistics
        for (int c = tid; c < kHeadGroup * (kKvDim / 8); c += kMlaThreads) {
            const int h = c / (kKvDim / 8), ch = c - h * (kKvDim / 8);
            const int head = hg * kHeadGroup + h;
            uint4 v = make_uint4(0, 0, 0, 0);
            if (head < a.heads) v = *reinterpret_cast<const uint4*>(qg + ((size_t)row * a.heads + head) * kKvDim + ch * 8);
            *reinterpret_cast<uint4*>(&sm.q[h][ch * 8]) = v;
        }
        if (tid < kHeadGroup) { sm.ml[tid][0] = -INFINITY; sm.ml[tid][1] = 0.f; }
        float o[8][4];  // warp w owns latent columns 64w .. 64w+63 of heads g and g + 8
#pragma unroll
        for (int n = 0; n < 8; ++n)
#pragma unroll
            for (int i = 0; i < 4; ++i) o[n][i] = 0.f;

        for (int ci = 0; ci < chunks; ++ci) {
            const int chunk = sp * chunks + ci;
            if (chunk >= total_chunks) break;
            __syncthreads();
            // ---- gather 64 cache rows, widen to bf16
            if (tid < kSplit) {
                const int kidx = chunk * kSplit + tid;
                int slot = kidx < a.topk ? a.topk_slots[(size_t)row * a.topk_ld + kidx] : -1;
                if (slot >= 0 && (int64_t)slot >= a.n_pages * kPage) slot = -1;
                sm.valid[tid] = slot;
            }
            __syncthreads();
            {
                constexpr int kChunks = kKvDim / 16;  // 36 sixteen-byte chunks per key
                constexpr int kPer = kSplit * kChunks / kMlaThreads;  // 9
                uint4 v[kPer];
                float sc[kPer];
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    const int c = tid + i * kMlaThreads;
                    const int key = c / kChunks, ch = c - key * kChunks;
                    const int slot = sm.valid[key];
                    if (slot >= 0) {
                        const uint8_t* page = a.kv_pages + (size_t)(slot / kPage) * kKvPageBytes;
                        const int off = slot % kPage;
                        v[i] = __ldg(reinterpret_cast<const uint4*>(page + (size_t)off * kKvDim) + ch);
                        sc[i] = __ldg(reinterpret_cast<const float*>(page + kPage * kKvDim) + off);
                    } else {
                        v[i] = make_uint4(0, 0, 0, 0);
                        sc[i] = 0.f;
                    }
                }
#pragma unroll
                for (int i = 0; i < kPer; ++i) {
                    const int c = tid + i * kMlaThreads;
                    const int key = c / kChunks, ch = c - key * kChunks;
                    e4m3x16_to_bf16(v[i], sc[i], &sm.kv[key][ch * 16]);
                }
            }
            __syncthreads();
            // ---- S = Q K^T: warp w owns keys 8w .. 8w+7; four accumulators over interleaved k steps keep the
            // MMAs independent of one another
            {
                float d[4][4];
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) d[i][j] = 0.f;
                const uint32_t q_addr = smem_u32(&sm.q[lane & 15][(lane >> 4) * 8]);
                const uint32_t k_addr = smem_u32(&sm.kv[warp * 8 + (lane & 7)][((lane >> 3) & 1) * 8]);
#pragma unroll
                for (int ks = 0; ks < kKvDim / 16; ks += 4) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        uint32_t af[4], bfr[2];
                        ldmatrix_x4(af, q_addr + (ks + u) * 32);
                        ldmatrix_x2(bfr, k_addr + (ks + u) * 32);
                        mma_bf16(d[u], af[0], af[1], af[2], af[3], bfr[0], bfr[1]);
                    }
                }
                float dd[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) dd[j] = (d[0][j] + d[1][j]) + (d[2][j] + d[3][j]);
                const int k0 = warp * 8 + 2 * t4;
                const bool v0 = sm.valid[k0] >= 0, v1 = sm.valid[k0 + 1] >= 0;
                sm.s[g][k0] = v0 ? dd[0] * a.sm_scale : -INFINITY;
                sm.s[g][k0 + 1] = v1 ? dd[1] * a.sm_scale : -INFINITY;
                sm.s[g + 8][k0] = v0 ? dd[2] * a.sm_scale : -INFINITY;
                sm.s[g + 8][k0 + 1] = v1 ? dd[3] * a.sm_scale : -INFINITY;
            }
            __syncthreads();
            // ---- running softmax: warp w owns heads 2w, 2w+1
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int h = warp * 2 + hh;
                const float s0 = sm.s[h][lane], s1 = sm.s[h][lane + 32];
                const float m_old = sm.ml[h][0];
                const float m = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
                const float p0 = (m == -INFINITY) ? 0.f : __expf(s0 - m);
                const float p1 = (m == -INFINITY) ? 0.f : __expf(s1 - m);
                const float rescale = (m == -INFINITY) ? 1.f : __expf(m_old - m);  // e^(-inf) = 0 for the first live chunk
                const float l = warp_sum(p0 + p1);
                sm.p[h][lane] = __float2bfloat16_rn(p0);
                sm.p[h][lane + 32] = __float2bfloat16_rn(p1);
                if (lane == 0) { sm.ml[h][0] = m; sm.ml[h][1] = sm.ml[h][1] * rescale + l; s_scale[h] = rescale; }
            }
            __syncthreads();
            // ---- O = O * rescale + P V
            {
                const float r0 = s_scale[g], r1 = s_scale[g + 8];
#pragma unroll
                for (int n = 0; n < 8; ++n) { o[n][0] *= r0; o[n][1] *= r0; o[n][2] *= r1; o[n][3] *= r1; }
                const uint32_t p_addr = smem_u32(&sm.p[lane & 15][(lane >> 4) * 8]);
#pragma unroll
                for (int ks = 0; ks < kSplit / 16; ++ks) {
                    uint32_t af[4];
                    ldmatrix_x4(af, p_addr + ks * 32);
#pragma unroll
                    for (int n2 = 0; n2 < 4; ++n2) {
                        // two n-tiles (16 columns) per x4.trans: matrices (k0..7,n0..7) (k8..15,n0..7) (k0..7,n8..15) (k8..15,n8..15)
                        uint32_t bfr[4];
                        const int krow = ks * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                        const int col = warp * 64 + n2 * 16 + (lane >> 4) * 8;
                        ldmatrix_x4_trans(bfr, smem_u32(&sm.kv[krow][col]));
                        mma_bf16(o[2 * n2], af[0], af[1], af[2], af[3], bfr[0], bfr[1]);
                        mma_bf16(o[2 * n2 + 1], af[0], af[1], af[2], af[3], bfr[2], bfr[3]);
                    }
                }
            }
        }
        __syncthreads();
        // ---- the task's partial: bf16 accumulator, f32 (m, l)
        {
            const int h0 = hg * kHeadGroup + g, h1 = h0 + 8;
#pragma unroll
            for (int n = 0; n < 8; ++n) {
                const int col = warp * 64 + n * 8 + 2 * t4;
                if (h0 < a.heads) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[n][0], o[n][1]);
                    *reinterpret_cast<__nv_bfloat162*>(part_acc + (((size_t)row * nsplit + sp) * a.heads + h0) * 512 + col) = v;
                }
                if (h1 < a.heads) {
                    __nv_bfloat162 v = __floats2bfloat162_rn(o[n][2], o[n][3]);
                    *reinterpret_cast<__nv_bfloat162*>(part_acc + (((size_t)row * nsplit + sp) * a.heads + h1) * 512 + col) = v;
                }
            }
            if (tid < kHeadGroup && hg * kHeadGroup + tid < a.heads) {
                float* ml = part_ml + (((size_t)row * nsplit + sp) * a.heads + hg * kHeadGroup + tid) * 2;
                ml[0] = sm.ml[tid][0];
                ml[1] = sm.ml[tid][1];
            }
        }
    }
}

// One CTA per (row, head): merge the splits.  With a destination in `q` the head's 512 merged values
// (rounded to bf16, as they are stored) are also quantised in place as the W_UV GEMV's activation set of
// that head: segment `head` of q.planes, four 128-value chunks, one warp each.
__global__ void __launch_bounds__(128) sparse_mla_merge_kernel(const mono_sparse_mla_args a, int nsplit, const mono_act_prep_args q) {
    pdl_prologue();
    __shared__ float w[128];
    __shared__ float merged[512];
    const int row = blockIdx.x / a.heads, head = blockIdx.x - row * a.heads;
    const __nv_bfloat16* part_acc = reinterpret_cast<const __nv_bfloat16*>(a.scratch);
    const float* part_ml = reinterpret_cast<const float*>(reinterpret_cast<const uint8_t*>(a.scratch) +
                                                          (size_t)a.rows * nsplit * a.heads * 512 * sizeof(__nv_bfloat16));
    const int tid = threadIdx.x;
    const int col = 4 * tid;
    // every thread requests its four columns of the first 32 partials before anything waits: the weights of
    // the splits (warp 0) and the partials arrive in the same memory latency
    constexpr int kBatch = 32;
    uint2 pv[kBatch];
#pragma unroll
    for (int j = 0; j < kBatch; ++j) {
        pv[j] = make_uint2(0u, 0u);
        if (j < nsplit)
            pv[j] = __ldcg(reinterpret_cast<const uint2*>(part_acc + (((size_t)row * nsplit + j) * a.heads + head) * 512 + col));
    }
    if (tid < 32) {
        float mx = -INFINITY;
        for (int j = tid; j < nsplit; j += 32) mx = fmaxf(mx, part_ml[(((size_t)row * nsplit + j) * a.heads + head) * 2]);
        mx = warp_max(mx);
        float den = 0.f;
        for (int j = tid; j < nsplit; j += 32) {
            const float* ml = part_ml + (((size_t)row * nsplit + j) * a.heads + head) * 2;
            const float e = (ml[0] == -INFINITY) ? 0.f : __expf(ml[0] - mx);
            w[j] = e;
            den += ml[1] * e;
        }
        den = warp_sum(den);
        __syncwarp();
        for (int j = tid; j < nsplit; j += 32) w[j] = den > 0.f ? w[j] / den : 0.f;
    }
    __syncthreads();
    float acc[4] = {0.f, 0.f, 0.f, 0.f};
    // a split without a live key has weight 0; whatever its accumulator holds must not reach the sum
    auto add = [&](const uint2& v, float wj) {
        if (wj == 0.f) return;
        const __nv_bfloat162 lo = *reinterpret_cast<const __nv_bfloat162*>(&v.x), hi = *reinterpret_cast<const __nv_bfloat162*>(&v.y);
        acc[0] += __low2float(lo) * wj;
        acc[1] += __high2float(lo) * wj;
        acc[2] += __low2float(hi) * wj;
        acc[3] += __high2float(hi) * wj;
    };
#pragma unroll
    for (int j = 0; j < kBatch; ++j)
        if (j < nsplit) add(pv[j], w[j]);
#pragma unroll 8
    for (int j = kBatch; j < nsplit; ++j)
        add(__ldcg(reinterpret_cast<const uint2*>(part_acc + (((size_t)row * nsplit + j) * a.heads + head) * 512 + col)), w[j]);
    const __nv_bfloat162 o01 = __floats2bfloat162_rn(acc[0], acc[1]), o23 = __floats2bfloat162_rn(acc[2], acc[3]);
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(a.out) + ((size_t)row * a.heads + head) * 512 + col) =
        make_uint2(*reinterpret_cast<const uint32_t*>(&o01), *reinterpret_cast<const uint32_t*>(&o23));
    if (q.planes) {
        merged[col] = __low2float(o01);
        merged[col + 1] = __high2float(o01);
        merged[col + 2] = __low2float(o23);
        merged[col + 3] = __high2float(o23);
        __syncthreads();
        const int warp = tid >> 5, lane = tid & 31;
        uint8_t* p0 = q.planes + (size_t)head * q.seg_stride + (size_t)row * q.ld;
        float* sf = q.scale_f32 ? q.scale_f32 + (size_t)head * q.scale_seg_stride + (size_t)row * q.scale_ld : nullptr;
        uint8_t* s8 = q.scale_e8 ? q.scale_e8 + (size_t)head * q.scale_seg_stride + (size_t)row * q.scale_ld : nullptr;
        quant_chunk128(merged + warp * 128, q.fmt, lane, warp, p0, p0 + q.plane_stride, sf, s8);
    }
}

}  // namespace mono

size_t mono_sparse_mla_tc_image_bytes(int rows);
int mono_sparse_mla_tc_split(const mono_sparse_mla_args* a, int nchunks, cudaStream_t st);

// From 64 local heads the split runs on tcgen05 with all heads of a row in one task (sparse_mla_tc.cu);
// MONO_MLA_TC=0 keeps the warp-MMA split (one task per 16 heads) for A/B measurements.
static bool mla_tc_wanted(int heads) {
    const char* e = getenv("MONO_MLA_TC");  // read at every launch: a test switches it inside one process
    return (e ? atoi(e) : 1) != 0 && heads >= 64;
}

extern "C" size_t mono_sparse_mla_scratch_bytes(int rows, int heads, int topk) {
    const size_t nsplit = (size_t)(topk + mono::kSplit - 1) / mono::kSplit;
    size_t n = (size_t)rows * nsplit * heads * (512 * sizeof(__nv_bfloat16) + 2 * sizeof(float)) + 256;
    if (heads >= 64) n = ((n + 1023) & ~size_t(1023)) + mono_sparse_mla_tc_image_bytes(rows);  // the query planes of the tcgen05 split
    return n;
}

// (nsplit, chunks per task): about two rounds of the resident CTAs (2 per SM) over rows x head groups x chunks
static void mla_plan(int rows, int heads, int topk, int sms, int* nsplit, int* chunks) {
    const int total = (topk + mono::kSplit - 1) / mono::kSplit;
    const int hgroups = (heads + mono::kHeadGroup - 1) / mono::kHeadGroup;
    const long work = (long)rows * hgroups * total;
    int c = (int)((work + 4L * sms - 1) / (4L * sms));
    c = c < 1 ? 1 : (c > 32 ? 32 : c);
    *chunks = c;
    *nsplit = (total + c - 1) / c;
}

static int sparse_mla_launch(const mono_sparse_mla_args* a, const mono_act_prep_args* dst, void* stream);

extern "C" int mono_sparse_mla_launch(const mono_sparse_mla_args* a, void* stream) { return sparse_mla_launch(a, nullptr, stream); }

extern "C" int mono_sparse_mla_quant_launch(const mono_sparse_mla_args* a, const mono_act_prep_args* dst, void* stream) {
    if (!a || !dst || !dst->planes || dst->rows != a->rows || dst->k != 512 || dst->segs != a->heads ||
        (dst->fmt == MONO_ACT_A8 && !dst->scale_f32) || (dst->fmt == MONO_ACT_HILO && (!dst->scale_f32 || dst->plane_stride <= 0)) ||
        ((dst->fmt == MONO_ACT_MX8 || dst->fmt == MONO_ACT_MX8N) && !dst->scale_e8)) {
        mono_set_error("mono_sparse_mla_quant_launch: the destination must describe rows x heads segments of 512 values "
                       "(k = 512, segs = heads) with planes and the scales of its format");
        return MONO_E_ARG;
    }
    return sparse_mla_launch(a, dst, stream);
}

static int sparse_mla_launch(const mono_sparse_mla_args* a, const mono_act_prep_args* dst, void* stream) {
    if (!a || a->rows < 1 || a->rows > MONO_MAX_ROWS || a->heads < 1 || a->heads > 128 || a->topk < 1 ||
        a->topk > 64 * 128 || a->topk_ld < a->topk || !a->q || !a->kv_pages || !a->topk_slots || !a->out || !a->scratch) {
        mono_set_error("mono_sparse_mla_launch: rows 1..16, heads 1..128, topk 1..8192 and all pointers required");
        return MONO_E_ARG;
    }
    if ((reinterpret_cast<uintptr_t>(a->kv_pages) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15) ||
        (reinterpret_cast<uintptr_t>(a->scratch) & 15)) {
        mono_set_error("mono_sparse_mla_launch: q, kv_pages and scratch must be 16-byte aligned");
        return MONO_E_ARG;
    }
    const int sms = mono_sm_count();
    int nsplit, chunks;
    if (mla_tc_wanted(a->heads)) {
        nsplit = (a->topk + mono::kSplit - 1) / mono::kSplit;
        if (int rc = mono_sparse_mla_tc_split(a, nsplit, (cudaStream_t)stream)) return rc;
        mono_act_prep_args none = {};
        mono::launch_k(mono::sparse_mla_merge_kernel, a->rows * a->heads, 128, 0, (cudaStream_t)stream, *a, nsplit, dst ? *dst : none);
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) mono_set_error("mono_sparse_mla_launch: %s", cudaGetErrorString(e));
        return (int)e;
    }
    mla_plan(a->rows, a->heads, a->topk, sms, &nsplit, &chunks);
    const size_t smem = sizeof(mono::MlaSmem) + 128;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(mono::sparse_mla_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            mono_set_error("mono_sparse_mla_launch: %s", cudaGetErrorString(e));
            return (int)e;
        }
        mono::attr_done(attr_once);
    }
    int grid = a->rows * ((a->heads + mono::kHeadGroup - 1) / mono::kHeadGroup) * nsplit;
    if (grid > 2 * sms) grid = 2 * sms;
    mono::launch_k(mono::sparse_mla_split_kernel, grid, mono::kMlaThreads, smem, (cudaStream_t)stream, *a, nsplit, chunks);
    mono_act_prep_args none = {};
    mono::launch_k(mono::sparse_mla_merge_kernel, a->rows * a->heads, 128, 0, (cudaStream_t)stream, *a, nsplit, dst ? *dst : none);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_sparse_mla_launch: %s", cudaGetErrorString(e));
    return (int)e;
}

// ------------------------------------------------------------------------------------
// Sparse MLA for callers that must not allocate.
//
// A serving process usually hands every free byte of the GPU to its KV-cache pool once
// the model is loaded, and from then on a late cudaMalloc can fail, fragment the pool's
// neighbourhood or stall the device while it maps memory; code that runs between graph
// captures, inside a latency-critical decode loop, or in a plugin that was attached
// after the pool was sized is in that position.  For those callers the split partials
// live in a fixed array that is part of the library image instead of a caller-provided
// scratch buffer.  Every GPU that loads the library holds the array until the process
// exits, so it is kept small: it covers steps of up to 8 rows x 16 local heads x 2048
// selected keys (the shape of BASELINE config 2); anything larger is refused.
//
// The array's name in host code is only a handle, not a device address, so the device
// address is looked up once per device with cudaGetSymbolAddress while that device is
// current, and that pointer is what the kernels receive.
namespace mono {
constexpr int kNoAllocRows = MONO_NOALLOC_MAX_ROWS, kNoAllocHeads = MONO_NOALLOC_MAX_HEADS,
              kNoAllocTopk = MONO_NOALLOC_MAX_TOPK;
constexpr size_t kNoAllocScratchBytes =
    (size_t)kNoAllocRows * (kNoAllocTopk / kSplit) * kNoAllocHeads * (512 * sizeof(__nv_bfloat16) + 2 * sizeof(float)) + 256;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];
}  // namespace mono

#include <mutex>

// Device address of the static scratch on the current device (nullptr + message on failure).
static void* noalloc_scratch_for_current_device() {
    constexpr int kMaxDevices = 64;
    static std::mutex mu;
    static void* ptrs[kMaxDevices] = {};
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess || dev < 0 || dev >= kMaxDevices) {
        mono_set_error("mono_sparse_mla_launch_noalloc: cudaGetDevice failed or device %d out of range (%s)", dev,
                       cudaGetErrorString(e));
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (ptrs[dev] == nullptr) {
        void* p = nullptr;
        e = cudaGetSymbolAddress(&p, mono::g_noalloc_scratch);
        if (e != cudaSuccess || p == nullptr) {
            mono_set_error("mono_sparse_mla_launch_noalloc: cudaGetSymbolAddress failed on device %d: %s", dev,
                           cudaGetErrorString(e));
            return nullptr;
        }
        ptrs[dev] = p;
    }
    return ptrs[dev];
}

extern "C" int mono_sparse_mla_launch_noalloc(const mono_sparse_mla_args* a, void* stream) {
    if (!a || a->rows < 1 || a->heads < 1 || a->topk < 1 || a->topk_ld < a->topk || !a->q || !a->kv_pages ||
        !a->topk_slots || !a->out) {
        mono_set_error("mono_sparse_mla_launch_noalloc: rows, heads, topk >= 1 and q, kv_pages, topk_slots, out required");
        return MONO_E_ARG;
    }
    if (a->rows > mono::kNoAllocRows || a->heads > mono::kNoAllocHeads || a->topk > mono::kNoAllocTopk) {
        mono_set_error("mono_sparse_mla_launch_noalloc: %d rows x %d heads x %d keys exceeds the built-in scratch "
                       "(at most %d x %d x %d); use mono_sparse_mla_launch with a caller-provided scratch buffer",
                       a->rows, a->heads, a->topk, mono::kNoAllocRows, mono::kNoAllocHeads, mono::kNoAllocTopk);
        return MONO_E_ARG;
    }
    if ((reinterpret_cast<uintptr_t>(a->kv_pages) & 15) || (reinterpret_cast<uintptr_t>(a->q) & 15)) {
        mono_set_error("mono_sparse_mla_launch_noalloc: q and kv_pages must be 16-byte aligned");
        return MONO_E_ARG;
    }
    void* scratch = noalloc_scratch_for_current_device();
    if (scratch == nullptr) return MONO_E_DRIVER;
    mono_sparse_mla_args args = *a;
    args.scratch = scratch;  // whatever the caller put there is ignored
    const int sms = mono_sm_count();
    if (sms <= 0) return MONO_E_DRIVER;
    int nsplit, chunks;
    mla_plan(args.rows, args.heads, args.topk, sms, &nsplit, &chunks);
    const size_t smem = sizeof(mono::MlaSmem) + 128;
    static std::atomic<uint64_t> attr_once{0};  // bit d: set on device d
    if (mono::attr_needed(attr_once)) {
        cudaError_t e = cudaFuncSetAttribute(mono::sparse_mla_split_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            mono_set_error("mono_sparse_mla_launch_noalloc: %s", cudaGetErrorString(e));
            return (int)e;
        }
        mono::attr_done(attr_once);
    }
    int grid = args.rows * ((args.heads + mono::kHeadGroup - 1) / mono::kHeadGroup) * nsplit;
    if (grid > 2 * sms) grid = 2 * sms;
    // Nothing in the scratch has to start at zero: every partial the merge reads is
    // written by this call's split kernel first (same stream, so in order).
    mono::sparse_mla_split_kernel<<<grid, mono::kMlaThreads, smem, (cudaStream_t)stream>>>(args, nsplit, chunks);
    mono_act_prep_args none = {};
    mono::sparse_mla_merge_kernel<<<args.rows * args.heads, 128, 0, (cudaStream_t)stream>>>(args, nsplit, none);
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) mono_set_error("mono_sparse_mla_launch_noalloc: %s", cudaGetErrorString(e));
    return (int)e;
}
