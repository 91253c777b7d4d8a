// Host-side plumbing of the C ABI: error strings, device queries, guard reads and
// TMA descriptor encoding.
#include <cstdarg>
#include <cstdio>
#include <cstring>

#include "mono_common.cuh"

static thread_local char g_err[512] = "";

void mono_set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

std::atomic<unsigned long long> g_mono_launches{0};
// Kernels this library has launched in this process (every launch goes through one helper): what a caller's
// "launches per step" claim is counted from.
extern "C" unsigned long long mono_launch_count(void) { return g_mono_launches.load(std::memory_order_relaxed); }

int g_mono_pdl = 1;
extern "C" int mono_set_pdl(int on) {
    const int old = g_mono_pdl;
    g_mono_pdl = on ? 1 : 0;
    return old;
}

extern "C" int mono_abi_version(void) { return MONO_ABI_VERSION; }
extern "C" const char* mono_last_error(void) { return g_err; }

extern "C" int mono_sm_count(void) {
    static thread_local int cached_dev = -1, cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) {
        mono_set_error("mono_sm_count: no CUDA device");
        return -1;
    }
    if (dev != cached_dev) {
        if (cudaDeviceGetAttribute(&cached, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -1;
        cached_dev = dev;
    }
    return cached;
}

extern "C" int mono_guard_read(const int32_t* guard_words, int32_t out[3], void* stream) {
    if (!guard_words || !out) {
        mono_set_error("mono_guard_read: null pointer");
        return MONO_E_ARG;
    }
    int32_t w[MONO_GUARD_WORDS];
    cudaError_t e = cudaMemcpyAsync(w, guard_words, sizeof(w), cudaMemcpyDeviceToHost, (cudaStream_t)stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e != cudaSuccess) {
        mono_set_error("mono_guard_read: %s", cudaGetErrorString(e));
        return (int)e;
    }
    out[0] = w[MONO_ERR_DEADLINE];
    out[1] = w[MONO_ERR_PEER];
    out[2] = w[MONO_ERR_ARG];
    if (out[0] | out[1] | out[2]) {
        mono_set_error("guard: deadline site %d, peer %d, arg site %d", out[0] - 1, out[1] - 1, out[2] - 1);
        return MONO_E_GUARD;
    }
    return 0;
}

// cuTensorMapEncodeTiled through the runtime's driver entry point (no -lcuda link).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

extern "C" int mono_tmap_encode_box(mono_tmap_t* out, const void* base, uint64_t inner_bytes, uint64_t rows,
                                    uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_rows);

extern "C" int mono_tmap_encode(mono_tmap_t* out, const void* base, uint64_t inner_bytes, uint64_t rows,
                                uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes) {
    return mono_tmap_encode_box(out, base, inner_bytes, rows, outer, row_stride_bytes, outer_stride_bytes, 128);
}

extern "C" int mono_tmap_encode_box(mono_tmap_t* out, const void* base, uint64_t inner_bytes, uint64_t rows,
                                    uint64_t outer, uint64_t row_stride_bytes, uint64_t outer_stride_bytes, uint32_t box_rows) {
    static_assert(sizeof(CUtensorMap) == sizeof(mono_tmap_t), "descriptor size");
    if (!out || !base || inner_bytes == 0 || rows == 0 || outer == 0 || box_rows == 0 || box_rows > 256) {
        mono_set_error("mono_tmap_encode: null or empty tensor, or box rows outside 1..256");
        return MONO_E_ARG;
    }
    if ((reinterpret_cast<uintptr_t>(base) & 15) || (row_stride_bytes & 15) || (outer_stride_bytes & 15) ||
        (inner_bytes & 15)) {
        mono_set_error("mono_tmap_encode: base, strides and row bytes must be multiples of 16 (base %p, row stride %llu)",
                       base, (unsigned long long)row_stride_bytes);
        return MONO_E_ARG;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        mono_set_error("mono_tmap_encode: cuTensorMapEncodeTiled not available from the driver");
        return MONO_E_DRIVER;
    }
    cuuint64_t dims[3] = {inner_bytes, rows, outer};
    cuuint64_t strides[2] = {row_stride_bytes, outer > 1 ? outer_stride_bytes : row_stride_bytes * rows};
    cuuint32_t box[3] = {128, box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        mono_set_error("mono_tmap_encode: cuTensorMapEncodeTiled failed with %d", (int)r);
        return MONO_E_DRIVER;
    }
    return 0;
}

extern "C" int mono_tmap_encode_fp4(mono_tmap_t* out, const void* base, uint64_t inner_elems, uint64_t rows, uint64_t outer,
                                    uint64_t row_stride_bytes, uint64_t outer_stride_bytes) {
    if (!out || !base || inner_elems == 0 || rows == 0 || outer == 0) {
        mono_set_error("mono_tmap_encode_fp4: null or empty tensor");
        return MONO_E_ARG;
    }
    // packed 4-bit tensors: 32-byte base, strides in multiples of 16 bytes, rows of whole 128-element boxes
    if ((reinterpret_cast<uintptr_t>(base) & 31) || (row_stride_bytes & 31) || (outer_stride_bytes & 31) || (inner_elems & 127)) {
        mono_set_error("mono_tmap_encode_fp4: base must be 32-byte aligned, strides multiples of 32 bytes, K a multiple of 128 "
                       "(base %p, row stride %llu, K %llu)", base, (unsigned long long)row_stride_bytes, (unsigned long long)inner_elems);
        return MONO_E_ARG;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        mono_set_error("mono_tmap_encode_fp4: cuTensorMapEncodeTiled not available from the driver");
        return MONO_E_DRIVER;
    }
    cuuint64_t dims[3] = {inner_elems, rows, outer};
    cuuint64_t strides[2] = {row_stride_bytes, outer > 1 ? outer_stride_bytes : row_stride_bytes * rows};
    cuuint32_t box[3] = {128, 128, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(reinterpret_cast<CUtensorMap*>(out), CU_TENSOR_MAP_DATA_TYPE_16U4_ALIGN16B, 3, const_cast<void*>(base), dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        mono_set_error("mono_tmap_encode_fp4: cuTensorMapEncodeTiled failed with %d", (int)r);
        return MONO_E_DRIVER;
    }
    return 0;
}

// ---- symmetric peer memory over CUDA IPC
extern "C" int mono_peer_alloc(size_t bytes, void** out_ptr) {
    if (!out_ptr || bytes == 0) {
        mono_set_error("mono_peer_alloc: null pointer or zero size");
        return MONO_E_ARG;
    }
    void* p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e == cudaSuccess) e = cudaMemset(p, 0, bytes);
    if (e == cudaSuccess) e = cudaDeviceSynchronize();
    if (e != cudaSuccess) {
        mono_set_error("mono_peer_alloc(%zu): %s", bytes, cudaGetErrorString(e));
        if (p) cudaFree(p);
        return (int)e;
    }
    *out_ptr = p;
    return 0;
}
extern "C" int mono_peer_export(void* ptr, unsigned char handle[MONO_IPC_HANDLE_BYTES]) {
    static_assert(sizeof(cudaIpcMemHandle_t) == MONO_IPC_HANDLE_BYTES, "IPC handle size");
    if (!ptr || !handle) return MONO_E_ARG;
    cudaIpcMemHandle_t h;
    cudaError_t e = cudaIpcGetMemHandle(&h, ptr);
    if (e != cudaSuccess) {
        mono_set_error("mono_peer_export: %s", cudaGetErrorString(e));
        return (int)e;
    }
    memcpy(handle, &h, sizeof(h));
    return 0;
}
extern "C" int mono_peer_open(const unsigned char handle[MONO_IPC_HANDLE_BYTES], void** out_ptr) {
    if (!handle || !out_ptr) return MONO_E_ARG;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle, sizeof(h));
    cudaError_t e = cudaIpcOpenMemHandle(out_ptr, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        mono_set_error("mono_peer_open: %s", cudaGetErrorString(e));
        return (int)e;
    }
    return 0;
}
extern "C" int mono_peer_close(void* opened_ptr) {
    if (!opened_ptr) return MONO_E_ARG;
    cudaError_t e = cudaIpcCloseMemHandle(opened_ptr);
    if (e != cudaSuccess) mono_set_error("mono_peer_close: %s", cudaGetErrorString(e));
    return (int)e;
}
extern "C" int mono_peer_free(void* ptr) {
    if (!ptr) return MONO_E_ARG;
    cudaError_t e = cudaFree(ptr);
    if (e != cudaSuccess) mono_set_error("mono_peer_free: %s", cudaGetErrorString(e));
    return (int)e;
}

// Copies `bytes` of a peer buffer (or any device memory of this process) to the host; blocks.  For tests and
// post-mortems that look at the (value, tag) words a step left behind.
extern "C" int mono_peer_read(void* dst_host, const void* src_device, size_t bytes) {
    if (!dst_host || !src_device || bytes == 0) return MONO_E_ARG;
    cudaError_t e = cudaDeviceSynchronize();
    if (e == cudaSuccess) e = cudaMemcpy(dst_host, src_device, bytes, cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) mono_set_error("mono_peer_read: %s", cudaGetErrorString(e));
    return (int)e;
}

extern "C" size_t mono_struct_size(int which) {
    switch (which) {
        case 0: return sizeof(mono_gemv_job);
        case 1: return sizeof(mono_gemv_args);
        case 2: return sizeof(mono_act_prep_args);
        case 3: return sizeof(mono_route_args);
        case 4: return sizeof(mono_mid_args);
        case 5: return sizeof(mono_sparse_mla_args);
        case 6: return sizeof(mono_reduce_args);
        case 7: return sizeof(mono_rowdot_args);
        case 8: return sizeof(mono_mla_mid_args);
        case 9: return sizeof(mono_q_post_args);
        case 10: return sizeof(mono_index_args);
        case 11: return sizeof(mono_gqa_args);
        case 12: return sizeof(mono_logits_gather_args);
        case 13: return sizeof(mono_prefetch_args);
        default: return 0;
    }
}
