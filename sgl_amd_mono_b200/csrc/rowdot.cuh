// The small row-dot GEMV's body, shared by the launches that run it (stages.cu: rowdot_kernel, router_kernel;
// attn_front.cu: index_prep_kernel).
#pragma once
#include "mono_common.cuh"

namespace mono {

// ------------------------------------------------------------------ small row-dot GEMV
// out[r][n] = sum_k x[r][k] * W[n][k] on CUDA cores, one warp per output column, for
// matrices too small to be worth a tensor-core launch (router logits with f32 or bf16
// weights: minimax_m31/ffn.py:601-649, glm53/gfx950/kernel.py:4199-4330).  The k
// order is fixed (lane-strided, then a butterfly), so every rank gets the same bits.
constexpr int kRowdotThreads = 256;

// Column n by the 256 threads tid = 0..255 of one group (every thread of the CTA calls this:
// it holds a CTA-wide barrier).  The weights do not depend on the launch before this one, so
// the first batch of weight loads is issued before the wait on that launch.
MONO_TL_DECLARE(tl_rowdot)
template <bool SMEM>
__device__ __forceinline__ uint2 ld_x(const __nv_bfloat16* p) {
    if (SMEM) {
        uint2 v;
        asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(smem_u32(p)));
        return v;
    }
    return __ldg(reinterpret_cast<const uint2*>(p));
}
#define COLS_GROUPS(c) 1  // rowdot_kernel: one 256-thread group per CTA calls rowdot_col
// `xs`: the step's activation rows staged in shared memory by the caller's CTA (one round trip for all of them), or
// NULL to read them from global memory as they are needed.
template <int COLS, bool STAGED = false>
__device__ __forceinline__ void rowdot_col(const mono_rowdot_args& a, int n0, int tid, float (*red)[kRowdotThreads / 32][kMaxRows],
                                           const __nv_bfloat16* xs = nullptr) {
    // columns n0 .. n0 + COLS - 1 share every activation load.  The 256 threads split K (4 values per
    // thread per 1024), so every weight load of a column is in flight at once; the order of the sums of
    // one column does not depend on COLS
    const int warp = tid >> 5, lane = tid & 31;
    float acc[COLS][kMaxRows];
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r) acc[c][r] = 0.f;
    const __nv_bfloat16* x = reinterpret_cast<const __nv_bfloat16*>(a.x_bf16);
    for (int k0 = 0; k0 < a.k; k0 += kRowdotThreads * 4 * 8) {
        // up to eight weight loads per thread and column are in flight before the first is used
        // (every load is unconditional, from a clamped address: a load under a condition is not issued before the
        // conversions of the one before it, and a column's weight loads would then cost a memory round trip each;
        // values past the matrix are zeroed after the loads)
        float4 wv[COLS][8];
        if (a.w_is_f32) {
#pragma unroll
            for (int c = 0; c < COLS; ++c)
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int k = k0 + (it * kRowdotThreads + tid) * 4;
                    wv[c][it] = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(a.w) + (size_t)min(n0 + c, a.n - 1) * a.k + min(k, a.k - 4)));
                }
        } else {
            uint2 raw[COLS][8];
#pragma unroll
            for (int c = 0; c < COLS; ++c)
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const int k = k0 + (it * kRowdotThreads + tid) * 4;
                    raw[c][it] = __ldg(reinterpret_cast<const uint2*>(reinterpret_cast<const __nv_bfloat16*>(a.w) + (size_t)min(n0 + c, a.n - 1) * a.k + min(k, a.k - 4)));
                }
#pragma unroll
            for (int c = 0; c < COLS; ++c)
#pragma unroll
                for (int it = 0; it < 8; ++it) {
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[c][it].x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw[c][it].y));
                    wv[c][it] = make_float4(lo.x, lo.y, hi.x, hi.y);
                }
        }
#pragma unroll
        for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int k = k0 + (it * kRowdotThreads + tid) * 4;
                if (!(k < a.k && n0 + c < a.n)) wv[c][it] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        if (k0 == 0) {
            MONO_TL(tl_rowdot, 1);
            pdl_wait();  // the activations come from the launch before this one
            MONO_TL(tl_rowdot, 2);
            if (STAGED) {
                // all rows into shared memory, every 16-byte piece requested at once
                const int pieces = a.rows * a.k / 8;
                for (int i = tid; i < pieces; i += kRowdotThreads * COLS_GROUPS(COLS))
                    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_u32(xs + (size_t)i * 8)), "l"(x + (size_t)i * 8) : "memory");
                asm volatile("cp.async.wait_all;" ::: "memory");
                __syncthreads();
                x = xs;
            }
            MONO_TL(tl_rowdot, 3);
        }
        // The activation loads of a batch (16 row x k-slice pairs) are all issued before the first is used:
        // one L2 round trip per batch instead of one per row.  A column's sums keep their order (k slice,
        // then row), so the bits do not depend on the batch shape.
        if (a.rows <= 8) {
#pragma unroll
            for (int it0 = 0; it0 < 8; it0 += 2) {
                uint2 xv[2][8];
#pragma unroll
                for (int h = 0; h < 2; ++h) {
                    const int k = k0 + ((it0 + h) * kRowdotThreads + tid) * 4;
#pragma unroll
                    for (int r = 0; r < 8; ++r)
                        xv[h][r] = ld_x<STAGED>(x + (size_t)min(r, a.rows - 1) * a.k + min(k, a.k - 4));
                }
                asm volatile("" ::: "memory");  // the next batch's loads start after this batch's, not among them
#pragma unroll
                for (int h = 0; h < 2; ++h)
#pragma unroll
                    for (int r = 0; r < 8; ++r) {
                        const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[h][r].x));
                        const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[h][r].y));
#pragma unroll
                        for (int c = 0; c < COLS; ++c)
                            acc[c][r] += lo.x * wv[c][it0 + h].x + lo.y * wv[c][it0 + h].y + hi.x * wv[c][it0 + h].z + hi.y * wv[c][it0 + h].w;
                    }
            }
        } else {
#pragma unroll
            for (int it = 0; it < 8; ++it) {
                const int k = k0 + (it * kRowdotThreads + tid) * 4;
                uint2 xv[kMaxRows];
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r)
                    xv[r] = ld_x<STAGED>(x + (size_t)min(r, a.rows - 1) * a.k + min(k, a.k - 4));
#pragma unroll
                for (int r = 0; r < kMaxRows; ++r) {
                    const float2 lo = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[r].x));
                    const float2 hi = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv[r].y));
#pragma unroll
                    for (int c = 0; c < COLS; ++c)
                        acc[c][r] += lo.x * wv[c][it].x + lo.y * wv[c][it].y + hi.x * wv[c][it].z + hi.y * wv[c][it].w;
                }
            }
        }
    }
    MONO_TL(tl_rowdot, 4);
#pragma unroll
    for (int c = 0; c < COLS; ++c)
#pragma unroll
        for (int r = 0; r < kMaxRows; ++r) {
            if (r < a.rows) {
                const float s = warp_sum(acc[c][r]);
                if (lane == 0) red[c][warp][r] = s;
            }
        }
    __syncthreads();
    if (tid < a.rows * COLS) {
        const int c = tid / a.rows, r = tid - c * a.rows;
        if (n0 + c < a.n) {
            float s = 0.f;
#pragma unroll
            for (int wv = 0; wv < kRowdotThreads / 32; ++wv) s += red[c][wv][r];
            a.out[(size_t)r * a.out_ld + n0 + c] = s * a.out_scale;
        }
    }
    MONO_TL(tl_rowdot, 5);
}

}  // namespace mono
