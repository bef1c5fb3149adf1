// Host side of the C ABI declared in include/nectarml_b200.h: turns a layer description into
// conversion passes, TMA tensor maps, a tile/phase/tap table and one launch of the
// contraction kernel.  No allocation, no synchronisation in the descriptor-based entry
// points; the reference-shaped entry points allocate their result as the reference does.
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <atomic>
#include <mutex>
#include <vector>

#include "../../include/nectarml_b200.h"
#include "nml_prepass.cuh"
#include "nml_umma.cuh"

namespace nml {

// ------------------------------------------------------------------ utilities --
#define NML_CUDA(expr)                                   \
    do {                                                 \
        cudaError_t e_ = (expr);                         \
        if (e_ != cudaSuccess) {                         \
            set_last_cuda_error(e_, #expr);              \
            return NML_ERR_CUDA;                         \
        }                                                \
    } while (0)

static thread_local char g_last_error[256] = {0};
static thread_local char g_last_scratch_error[256] = {0};
static thread_local char g_last_device_error[96] = {0};
static void set_last_cuda_error(cudaError_t e, const char* what) {
    snprintf(g_last_error, sizeof(g_last_error), "%s: %s", what, cudaGetErrorString(e));
}

static inline size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
static inline int ceil_div(int a, int b) { return (a + b - 1) / b; }

struct DeviceState;

// Bump allocator over the caller's workspace; in dry mode it only measures.
struct Bump {
    uint8_t* base;
    size_t off, cap;
    bool dry;
    DeviceState* ds = nullptr;  // when set, used instead of the lazily allocated per-device state
    void* take(size_t bytes) {
        off = round_up(off, 256);
        void* p = dry ? nullptr : base + off;
        off += bytes;
        return p;
    }
    bool fits() const { return dry || off <= cap; }
};

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn get_encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Tuning overrides for experiments and A/B measurements, read from the environment ONCE, when the
// library is first used (unset in normal use; every default is the measured-best setting):
//   NML_TUNE_STAGES   cap on the ring depth            NML_TUNE_BN        forced tile width (64 / 128 / 256)
//   NML_TUNE_KA       K atoms per stage (1 or 2)       NML_TUNE_L2PROMO   TMA L2 promotion (0..3)
//   NML_TUNE_PAIR     0: no CTA pairs                  NML_TUNE_TMASTORE  0: no TMA-store epilogues
//   NML_TUNE_EPI8     0: never a second epilogue group NML_TUNE_EPI8_K    K slices up to which it is used
//   NML_TUNE_PATCH    0: no forward patch walk, 2: wherever it is legal, 3: also with streamed weights
//   NML_TUNE_BRES     0: patch walk streams its weights NML_TUNE_SHUFFLE  0: no phase-packed gather walk
//   NML_TUNE_FSPLIT   0: no K split of the forward walk
//   NML_TUNE_WPATCH   0: no weight-gradient patch walk NML_TUNE_WCOAL     0: its gradient leaves by scattered stores
//   NML_TUNE_WTRANS   0: Linear input-gradients never take a transposed copy of the weights
//   NML_TUNE_PAIR128  0: CTA pairs only for 256-column tiles
struct Tune {
    int stages, bn, ka, l2promo, pair, tmastore, epi8, epi8_k, patch, bres, shuffle, fsplit, wpatch, wcoal, wtrans, pair128;
};
static const Tune& tune() {
    static Tune t;
    static std::once_flag once;
    std::call_once(once, [] {
        auto env = [](const char* name, int dflt) {
            const char* v = getenv(name);
            return (v && *v) ? atoi(v) : dflt;
        };
        t.stages = env("NML_TUNE_STAGES", 8);
        t.bn = env("NML_TUNE_BN", 0);
        t.ka = env("NML_TUNE_KA", 0);  // 0: chosen per launch
        t.l2promo = env("NML_TUNE_L2PROMO", 3);
        t.pair = env("NML_TUNE_PAIR", 1);
        t.tmastore = env("NML_TUNE_TMASTORE", 1);
        t.epi8 = env("NML_TUNE_EPI8", 1);
        t.epi8_k = env("NML_TUNE_EPI8_K", 8);
        t.patch = env("NML_TUNE_PATCH", 1);
        t.bres = env("NML_TUNE_BRES", 1);
        t.shuffle = env("NML_TUNE_SHUFFLE", 1);
        t.fsplit = env("NML_TUNE_FSPLIT", 1);
        t.wpatch = env("NML_TUNE_WPATCH", 1);
        t.wcoal = env("NML_TUNE_WCOAL", 1);
        t.wtrans = env("NML_TUNE_WTRANS", 1);
        t.pair128 = env("NML_TUNE_PAIR128", 1);
    });
    return t;
}

enum { SWZ_NONE = 0, SWZ_128B = 1, SWZ_128B_ATOM32 = 2 };

// Tensor map over a dense tensor given fastest-first dims; strides are the dense ones.
static int encode_map(CUtensorMap* tm, const void* ptr, int elem_bytes, int rank, const uint64_t* dims,
                      const uint32_t* box, const uint32_t* estr, int swizzle,
                      const uint64_t* stride_bytes = nullptr) {
    EncodeTiledFn fn = get_encode_fn();
    if (!fn) {
        snprintf(g_last_error, sizeof(g_last_error), "cuTensorMapEncodeTiled not available");
        return NML_ERR_CUDA;
    }
    cuuint64_t gdim[5], gstr[5];
    cuuint32_t b[5], es[5];
    uint64_t pitch = elem_bytes;
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        b[i] = box[i];
        es[i] = estr[i];
        pitch *= dims[i];
        if (i + 1 < rank) gstr[i] = stride_bytes ? stride_bytes[i] : pitch;  // stride of dim i+1
    }
    CUresult r = fn(tm, elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                    rank, const_cast<void*>(ptr), gdim, gstr, b, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    swizzle == SWZ_128B ? CU_TENSOR_MAP_SWIZZLE_128B
                    : swizzle == SWZ_128B_ATOM32 ? CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B
                                                 : CU_TENSOR_MAP_SWIZZLE_NONE,
                    static_cast<CUtensorMapL2promotion>(tune().l2promo),
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        snprintf(g_last_error, sizeof(g_last_error),
                 "cuTensorMapEncodeTiled failed (%d): rank %d dims %llu %llu %llu %llu box %u %u %u %u",
                 (int)r, rank, (unsigned long long)dims[0], (unsigned long long)(rank > 1 ? dims[1] : 0),
                 (unsigned long long)(rank > 2 ? dims[2] : 0), (unsigned long long)(rank > 3 ? dims[3] : 0),
                 box[0], rank > 1 ? box[1] : 0, rank > 2 ? box[2] : 0, rank > 3 ? box[3] : 0);
        return NML_ERR_CUDA;
    }
    return NML_OK;
}

// Per-device state: status word the kernels report into, SM count.
struct DeviceState {
    int* err = nullptr;
    int sms = 0;
    bool attr_set = false;
};
static DeviceState g_dev[64];
static std::mutex g_dev_mutex;   // guards g_dev, g_static, g_prof and g_ref_ws
static std::atomic<long long> g_launches{0};
// Where kernels report an abandoned wait.  The words live in the library image, so set-up needs no
// allocation: their device addresses come from cudaGetSymbolAddress, once per device.
static __device__ int g_status_word;
// Per-launch overrides used by the nml_debug_* entry points only (0 / false in normal use).
static thread_local unsigned long long g_dbg_wait_limit_ns = 0;
static thread_local bool g_dbg_short_a_box = false;

struct Profiler {
    std::atomic<bool> on{false};
    int cap = 0, n = 0;
    std::vector<cudaEvent_t> start, stop;
};
static Profiler g_prof;

// The instances of the contraction kernel, and the one that serves a given launch.
typedef void (*UmmaKernel)(const KParams);
template <int kOut, bool kPair>
static UmmaKernel fprop_instance(bool f16) {
    return f16 ? umma_conv_kernel<MODE_FPROP, kOut, true, kPair> : umma_conv_kernel<MODE_FPROP, kOut, false, kPair>;
}
static UmmaKernel kernel_for(const KParams& P) {
    if (P.mode == MODE_WGRAD)
        return P.pair ? umma_conv_kernel<MODE_WGRAD, OUT_NHWC, false, true> : umma_conv_kernel<MODE_WGRAD, OUT_NHWC, false, false>;
    const bool h = P.out_f16 != 0;
    if (P.pair) {
        if (P.out_mode == OUT_NHWC_TMA) return fprop_instance<OUT_NHWC_TMA, true>(h);
        if (P.out_mode == OUT_NCHW_TMA) return fprop_instance<OUT_NCHW_TMA, true>(h);
        return fprop_instance<OUT_NCHW, true>(h);
    }
    if (P.out_mode == OUT_NHWC_TMA) return fprop_instance<OUT_NHWC_TMA, false>(h);
    if (P.out_mode == OUT_NCHW_TMA) return fprop_instance<OUT_NCHW_TMA, false>(h);
    if (P.out_mode == OUT_NHWC) return fprop_instance<OUT_NHWC, false>(h);
    return fprop_instance<OUT_NCHW, false>(h);
}
static int raise_smem_limit() {
    UmmaKernel all[16] = {umma_conv_kernel<MODE_WGRAD, OUT_NHWC, false, false>, umma_conv_kernel<MODE_WGRAD, OUT_NHWC, false, true>,
                          fprop_instance<OUT_NHWC_TMA, false>(true), fprop_instance<OUT_NHWC_TMA, false>(false),
                          fprop_instance<OUT_NCHW_TMA, false>(true), fprop_instance<OUT_NCHW_TMA, false>(false),
                          fprop_instance<OUT_NHWC, false>(true), fprop_instance<OUT_NHWC, false>(false),
                          fprop_instance<OUT_NCHW, false>(true), fprop_instance<OUT_NCHW, false>(false),
                          fprop_instance<OUT_NHWC_TMA, true>(true), fprop_instance<OUT_NHWC_TMA, true>(false),
                          fprop_instance<OUT_NCHW_TMA, true>(true), fprop_instance<OUT_NCHW_TMA, true>(false),
                          fprop_instance<OUT_NCHW, true>(true), fprop_instance<OUT_NCHW, true>(false)};
    for (UmmaKernel k : all)
        NML_CUDA(cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 232448));
    return NML_OK;
}

// Loads every helper kernel of the library (with lazy module loading a kernel is otherwise loaded by
// its first launch, which may allocate and must not happen inside a stream capture).
static int load_helper_kernels() {
    const void* fns[] = {
        (const void*)nchw_to_nhwc_kernel<float>, (const void*)nchw_to_nhwc_kernel<__half>,
        (const void*)convert_rows_kernel<float>, (const void*)convert_rows_kernel<__half>,
        (const void*)colsum_rows_kernel<float>, (const void*)colsum_rows_kernel<__half>,
        (const void*)colsum_rows_f16x8_kernel,
        (const void*)repack_weight_tile_kernel<float>, (const void*)repack_weight_tile_kernel<__half>,
        (const void*)repack_weight_rows_kernel<float>, (const void*)repack_weight_rows_kernel<__half>,
        (const void*)pad_pack_c8_kernel<float>, (const void*)pad_pack_c8_kernel<__half>,
        (const void*)repack_weight_c8_kernel<float>, (const void*)repack_weight_c8_kernel<__half>,
        (const void*)finish_rows_kernel<float>, (const void*)finish_rows_kernel<__half>,
        (const void*)pack_phase_weights_kernel<float, float>, (const void*)pack_phase_weights_kernel<float, __half>,
        (const void*)pack_phase_weights_kernel<__half, float>, (const void*)pack_phase_weights_kernel<__half, __half>,
        (const void*)to_float_kernel<__half>, (const void*)colsum_finish_kernel,
        (const void*)wgrad_reduce_rows4_kernel, (const void*)wgrad_reduce_kernel, (const void*)wgrad_reduce_deep4_kernel,
    };
    for (const void* f : fns) {
        cudaFuncAttributes a;
        NML_CUDA(cudaFuncGetAttributes(&a, f));
    }
    return NML_OK;
}

// One-time set-up of the current device (first use, or nml_init): looks up the status word, loads the
// kernels and raises their shared-memory limit.  Allocates nothing; the cudaMemset is synchronous.
static int device_state(DeviceState** out) {
    int dev = 0;
    NML_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NML_ERR_INVALID;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    DeviceState& s = g_dev[dev];
    if (!s.attr_set) {
        void* status = nullptr;
        NML_CUDA(cudaGetSymbolAddress(&status, g_status_word));
        NML_CUDA(cudaMemset(status, 0, sizeof(int)));
        NML_CUDA(cudaDeviceGetAttribute(&s.sms, cudaDevAttrMultiProcessorCount, dev));
        int rc_attr = raise_smem_limit();
        if (rc_attr) return rc_attr;
        rc_attr = load_helper_kernels();
        if (rc_attr) return rc_attr;
        s.err = static_cast<int*>(status);
        s.attr_set = true;
    }
    *out = &s;
    return NML_OK;
}

// Upper bound on the SMs a launch may occupy (nml_set_sm_limit); 0 = all of them.
static std::atomic<int> g_sm_limit{0};
static inline int limited(int sms) {
    const int lim = g_sm_limit.load(std::memory_order_relaxed);
    return (lim > 0 && lim < sms) ? lim : sms;
}
// SM count the planner assumes: the current device's, or a B200's 148 where no device is present
// (workspace-size queries work on a machine without a GPU).
static int planning_sms() {
    static std::atomic<int> cached{0};
    int v = cached.load();
    if (v > 0) return limited(v);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
        sms <= 0) {
        (void)cudaGetLastError();
        return limited(148);
    }
    cached.store(sms);
    return limited(sms);
}

struct MathInfo {
    int es, kb, enc, planes, kind;
};
static bool math_info(int math, MathInfo* m) {
    switch (math) {
        case NML_MATH_F16: *m = {2, 64, ENC_F16, 1, KIND_F16}; return true;
        case NML_MATH_3XTF32: *m = {4, 32, ENC_TF32_PAIR, 2, KIND_TF32}; return true;
        case NML_MATH_TF32: *m = {4, 32, ENC_TF32_HI, 1, KIND_TF32}; return true;
    }
    return false;
}

// Bias gradient = column sums of dY, in two stages so that the result is bitwise repeatable: the pass
// that reads dY writes rows of partial sums ([P][stride], one row per block), colsum_finish_kernel adds
// the rows in a fixed order.  Both scratch matrices come from the workspace.
struct ColsumScratch {
    float* partial = nullptr;
    float* second = nullptr;
    int P = 0, stride = 0;
};
static ColsumScratch colsum_scratch(Bump& ws, size_t P, int stride) {
    ColsumScratch c;
    c.P = static_cast<int>(P);
    c.stride = stride;
    c.partial = static_cast<float*>(ws.take(P * stride * sizeof(float)));
    if (P > 256) c.second = static_cast<float*>(ws.take(((P + 255) / 256) * stride * sizeof(float)));
    return c;
}
static int colsum_finish(const ColsumScratch& cs, int C, float* out, cudaStream_t st) {
    const float* src = cs.partial;
    int P = cs.P, stride = cs.stride;
    for (;;) {
        const int S = ceil_div(P, 256);
        float* dst = (S == 1) ? out : (src == cs.partial ? cs.second : cs.partial);
        colsum_finish_kernel<<<dim3(ceil_div(C, 32), S), dim3(32, 8), 0, st>>>(src, P, stride, C, dst, cs.stride, 256);
        ++g_launches;
        if (S == 1) break;
        src = dst;
        P = S;
        stride = cs.stride;
    }
    NML_CUDA(cudaGetLastError());
    return NML_OK;
}

// Converts an activation tensor into the NHWC operand encoding of `mi` unless it already is one.
// planes[0..1] receive the operand pointers, *cp the padded channel count.  With `colsum` the
// per-channel sums of the tensor (the bias gradient) are produced in the same pass where there is one.
static int prepare_activation(const void* src, int dtype, int layout, int batch, int c, int h, int w,
                              const MathInfo& mi, Bump& ws, cudaStream_t st, const void* planes[2], int* cp,
                              float* colsum) {
    const int align = 16 / mi.es;
    const bool direct = (mi.enc == ENC_F16) && dtype == NML_F16 && (c % align == 0) &&
                        (layout == NML_NHWC || (h == 1 && w == 1) || c == 1);
    const size_t pixels = static_cast<size_t>(batch) * h * w;
    // row-major column sums: enough row blocks to fill the GPU, few enough that the second stage stays negligible
    const int col_blocks = ceil_div(c, 256);
    const int rows_per_block = static_cast<int>(std::max<size_t>(64, round_up(ceil_div(static_cast<int>(std::min<size_t>(pixels, 1u << 30)), std::max(1, 1184 / col_blocks)), 8)));
    const size_t row_blocks = (pixels + rows_per_block - 1) / rows_per_block;
    auto rows_colsum = [&](const ColsumScratch& cs) -> int {
        dim3 grid(col_blocks, static_cast<unsigned>(row_blocks));
        if (dtype == NML_F16 && c % 8 == 0 && (reinterpret_cast<uintptr_t>(src) & 15) == 0)
            colsum_rows_f16x8_kernel<<<grid, 256, 0, st>>>(static_cast<const __half*>(src), cs.partial, pixels, c, rows_per_block);
        else if (dtype == NML_F16)
            colsum_rows_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(src), cs.partial, pixels, c, rows_per_block);
        else
            colsum_rows_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), cs.partial, pixels, c, rows_per_block);
        ++g_launches;
        return colsum_finish(cs, c, colsum, st);
    };
    if (direct) {
        planes[0] = src;
        planes[1] = nullptr;
        *cp = c;
        if (colsum) {
            ColsumScratch cs = colsum_scratch(ws, row_blocks, c);
            if (ws.dry) return NML_OK;
            if (!ws.fits()) return NML_ERR_WORKSPACE;
            return rows_colsum(cs);
        }
        return NML_OK;
    }
    const int Cp = static_cast<int>(round_up(c, align));
    *cp = Cp;
    void* p0 = ws.take(pixels * Cp * mi.es);
    void* p1 = (mi.planes == 2) ? ws.take(pixels * Cp * mi.es) : nullptr;
    planes[0] = p0;
    planes[1] = p1;
    const bool transposing = layout == NML_NCHW && !(h == 1 && w == 1);
    ColsumScratch cs;
    if (colsum) cs = transposing ? colsum_scratch(ws, static_cast<size_t>(batch) * ceil_div(h * w, 64), c) : colsum_scratch(ws, row_blocks, c);
    if (ws.dry) return NML_OK;
    if (!ws.fits()) return NML_ERR_WORKSPACE;
    if (transposing) {
        dim3 grid(ceil_div(h * w, 64), ceil_div(Cp, 64), batch);
        if (dtype == NML_F32)
            { nchw_to_nhwc_kernel<float><<<grid, 256, 0, st>>>(static_cast<const float*>(src), p0, p1, mi.enc, c, Cp,
                                                            h * w, cs.partial); ++g_launches; }
        else
            { nchw_to_nhwc_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(src), p0, p1, mi.enc, c,
                                                             Cp, h * w, cs.partial); ++g_launches; }
        if (colsum) {
            int rc = colsum_finish(cs, c, colsum, st);
            if (rc) return rc;
        }
    } else {
        size_t total = pixels * Cp;
        int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 16));
        if (dtype == NML_F32)
            { convert_rows_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(src), p0, p1, mi.enc, pixels,
                                                              c, Cp); ++g_launches; }
        else
            { convert_rows_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(src), p0, p1, mi.enc,
                                                               pixels, c, Cp); ++g_launches; }
        if (colsum) {
            int rc = rows_colsum(cs);
            if (rc) return rc;
        }
    }
    NML_CUDA(cudaGetLastError());
    return NML_OK;
}

// Few-channel path: the activation as a zero-padded [N][Hp][Wp][8] fp16 image (see pad_pack_c8_kernel).
// Wp leaves room for the 8-pixel window of the last output column.
struct WindowImage {
    const void* ptr;
    int hp, wp;
};
static bool window_eligible(int c, int kw, int d_w, int enc) { return c <= 8 && kw <= 8 && d_w == 1 && enc == ENC_F16; }
static int prepare_window(const void* src, int dtype, int layout, int batch, int c, int h, int w, int p_h, int p_w,
                          int s_w, int out_w, Bump& ws, cudaStream_t st, WindowImage* img, float* colsum = nullptr) {
    img->hp = h + 2 * p_h;
    img->wp = std::max(w + 2 * p_w, (out_w - 1) * s_w + 8);
    const size_t pixels = static_cast<size_t>(batch) * img->hp * img->wp;
    void* p = ws.take(pixels * 16);
    img->ptr = p;
    int blocks = static_cast<int>(std::min<size_t>((pixels + 255) / 256, 148 * 32));
    ColsumScratch cs;
    if (colsum) cs = colsum_scratch(ws, blocks, 8);  // one row of 8 channel sums per block
    if (ws.dry) return NML_OK;
    if (!ws.fits()) return NML_ERR_WORKSPACE;
    const int nchw = (layout == NML_NCHW) ? 1 : 0;
    if (dtype == NML_F32)
        { pad_pack_c8_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(src), nchw, static_cast<__half*>(p), batch, c, h, w, p_h, p_w, img->hp, img->wp, cs.partial); ++g_launches; }
    else
        { pad_pack_c8_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(src), nchw, static_cast<__half*>(p), batch, c, h, w, p_h, p_w, img->hp, img->wp, cs.partial); ++g_launches; }
    NML_CUDA(cudaGetLastError());
    if (colsum) return colsum_finish(cs, c, colsum, st);
    return NML_OK;
}

// Picks a power-of-two pixel box (w, h, n) with 2^bits pixels that covers the grid with the
// fewest boxes; ties go to the wider box.  box extents times the element stride stay <= 256.
static void choose_box(int bits, int gw, int gh, int gn, int s_w, int s_h, int* wl, int* hl, int* nl,
                       int prefer_w_log2 = 0) {
    long long best = -1, best_wide = -1;
    int ww = 0, wh = 0, wn = 0;
    for (int a = bits; a >= 0; --a) {
        if ((1 << a) * s_w > 256) continue;
        for (int b = bits - a; b >= 0; --b) {
            if ((1 << b) * s_h > 256) continue;
            int c = bits - a - b;
            if ((1 << c) > 256) continue;
            long long tiles = 1ll * ceil_div(gw, 1 << a) * ceil_div(gh, 1 << b) * ceil_div(gn, 1 << c);
            if (best < 0 || tiles < best) {
                best = tiles;
                *wl = a;
                *hl = b;
                *nl = c;
            }
            if (a >= prefer_w_log2 && (best_wide < 0 || tiles < best_wide)) {
                best_wide = tiles;
                ww = a;
                wh = b;
                wn = c;
            }
        }
    }
    // A box at least 2^prefer_w_log2 pixels wide (whole 128-byte runs for pixel-major stores) is taken
    // when it costs at most 15 % more tiles.
    if (prefer_w_log2 > 0 && best_wide > 0 && best_wide * 100 <= best * 115) {
        *wl = ww;
        *hl = wh;
        *nl = wn;
    }
}


// Closes the timing bracket of a recorded launch (see nml_profile_begin).
static int profile_stop(int slot, cudaStream_t st) {
    if (slot >= 0) NML_CUDA(cudaEventRecord(g_prof.stop[slot], st));
    return NML_OK;
}

// Launches the contraction kernel.  When `open_slot` is given and the launch is being timed, the
// bracket is left open (slot index returned there) so that the caller can include the kernel's
// second-stage reduction; the caller then closes it with profile_stop.
// Opens a timing bracket before a pass's preparatory kernels (so that they are counted in the pass's
// duration); launch_kernel then continues that bracket instead of opening its own.
static thread_local int g_bracket_slot = -1;
static int profile_open(cudaStream_t st) {
    if (!g_prof.on.load(std::memory_order_relaxed)) return NML_OK;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    if (g_prof.on.load() && g_prof.n < g_prof.cap) {
        g_bracket_slot = g_prof.n++;
        NML_CUDA(cudaEventRecord(g_prof.start[g_bracket_slot], st));
    }
    return NML_OK;
}

static int launch_kernel(KParams& P, DeviceState* ds, cudaStream_t st, int* open_slot = nullptr) {
    // Narrow tiles finish a 64-deep K slice in well under the barrier round trip of a stage, so they
    // take two slices per stage (8 MMAs per round trip); 256-wide tiles already fill 512 clocks.
    P.ka = (P.pair && P.bn == 256) ? 1 : std::max(1, std::min(2, tune().ka ? tune().ka : (P.bn >= 192 ? 1 : 2)));
    const int stage_bytes = P.ka * (kStageABytes + (P.pair ? P.bn / 2 : P.bn) * 128);
    // Shared memory: the operand ring, then the epilogue's staging buffers (two per warp if that does not
    // cost a ring stage, else one), the per-warp bias tiles, and the barriers.
    const int fixed = 1024 + 256 + kBiasTileBytes;
    const bool tma_out = (P.mode == MODE_FPROP) && NML_IS_TMA_OUT(P.out_mode);
    // A second group of four epilogue warps (TMA-store instances only) halves the drain time of a tile;
    // it pays where the K loop is too short to hide the drain behind the next tile's MMAs.
    {
        const int cpi = P.out_f16 ? 64 : 32;
        int k_slices = 0;  // 64-deep (fp16) K slices per tile, longest phase
        for (int p = 0; p < P.n_phases; ++p) k_slices = std::max(k_slices, P.passes * P.c_blocks * P.phases[p].tap_count);
        const bool short_k = k_slices <= tune().epi8_k;
        P.epi_warps = (tma_out && short_k && P.bn / cpi >= 2 && tune().epi8) ? 8 : 4;
    }
    size_t smem;
    if (P.wpatch) {
        // [stages x (patch, box of the other tensor)][staging (unused by this walk)][bias][barriers]
        P.ka = 1;
        P.epi_warps = 4;
        P.stg_bufs = 1;
        const int w_stage = P.patch_bytes + P.bn * 128;
        const int avail = 232448 - fixed - P.epi_warps * P.stg_bufs * kStagingBufBytes;
        P.stages = std::max(2, std::min(8, avail / w_stage));
        P.ring_bytes = P.stages * w_stage;
        {
            const long long run = 1ll * P.c_patch * P.n_taps * (P.kw_pack ? P.kw_count : 1);
            P.w_coalesce = (tune().wcoal && 32 * run * 4 <= P.ring_bytes && P.num_tiles <= limited(ds->sms)) ? 1 : 0;
        }
        smem = static_cast<size_t>(P.ring_bytes) + P.epi_warps * P.stg_bufs * kStagingBufBytes + fixed;
    } else if (P.patch) {
        // [B: resident slices, or a ring of single-slice stages][patch buffers][staging][bias][barriers]
        P.ka = 1;
        const int b_slice = P.bn * 128;
        const int res_bytes = P.c_blocks * P.n_taps * b_slice;  // the taps of every phase
        P.stg_bufs = 2;
        int avail = 232448 - fixed - P.epi_warps * P.stg_bufs * kStagingBufBytes;
        const bool res_wanted = P.n_tiles == 1 && P.passes == 1 && tune().bres;
        if (res_wanted && res_bytes + 2 * P.patch_bytes > avail) {  // trade staging for residency
            P.stg_bufs = 1;
            avail = 232448 - fixed - P.epi_warps * P.stg_bufs * kStagingBufBytes;
            if (res_bytes + 2 * P.patch_bytes > avail) {
                P.epi_warps = 4;
                avail = 232448 - fixed - P.epi_warps * P.stg_bufs * kStagingBufBytes;
            }
        }
        int b_region;
        if (res_wanted && res_bytes + 2 * P.patch_bytes <= avail) {
            P.b_resident = 1;
            P.stages = 1;
            b_region = res_bytes;
            P.a_stages = std::min(4, (avail - res_bytes) / P.patch_bytes);
        } else {
            P.b_resident = 0;
            // B streams tap by tap; narrow tiles take two taps per stage (8 MMAs per barrier round trip)
            P.ka = std::max(1, std::min(2, tune().ka ? tune().ka : (P.bn >= 192 ? 1 : 2)));
            const int b_stage = P.ka * b_slice;
            P.a_stages = std::min(3, std::max(2, P.passes * P.c_blocks));
            P.stages = std::min(8, (avail - P.a_stages * P.patch_bytes) / b_stage);
            if (P.stages < 3) {  // wide tiles: give the B ring room
                P.a_stages = 2;
                P.stg_bufs = 1;
                avail = 232448 - fixed - P.epi_warps * P.stg_bufs * kStagingBufBytes;
                P.stages = std::min(8, (avail - P.a_stages * P.patch_bytes) / b_stage);
            }
            if (P.stages < 2) return NML_ERR_UNSUPPORTED;
            b_region = P.stages * b_stage;
        }
        P.issuers = (P.b_resident && P.a_stages >= 2 * P.c_blocks) ? 2 : 1;
        P.a_ring_off = static_cast<int>(round_up(b_region, 1024));
        P.ring_bytes = P.a_ring_off + P.a_stages * P.patch_bytes;
        smem = static_cast<size_t>(P.ring_bytes) + P.epi_warps * P.stg_bufs * kStagingBufBytes + fixed;
    } else {
    int stages2 = (232448 - fixed - P.epi_warps * 2 * kStagingBufBytes) / stage_bytes;
    int stages1 = (232448 - fixed - P.epi_warps * 1 * kStagingBufBytes) / stage_bytes;
    P.stg_bufs = (stages2 >= std::min(stages1, 8)) ? 2 : 1;
    int stages = std::min(8, P.stg_bufs == 2 ? stages2 : stages1);
    stages = std::max(2, std::min(stages, tune().stages));
    P.stages = stages;
    P.ring_bytes = stages * stage_bytes;
    smem = static_cast<size_t>(stages) * stage_bytes + P.epi_warps * P.stg_bufs * kStagingBufBytes + fixed;
    }
    smem = std::max<size_t>(smem, 120 * 1024);  // one CTA per SM: each allocates its own TMEM
    P.err = ds->err;
    int grid = P.pair ? 2 * std::min(P.num_tiles, limited(ds->sms) / 2) : std::min(P.num_tiles, limited(ds->sms));
    if (grid <= 0) return NML_OK;
    P.wait_limit_ns = g_dbg_wait_limit_ns;
    int rec_slot = g_bracket_slot;  // a bracket the caller opened, if any
    g_bracket_slot = -1;
    const bool pre_opened = rec_slot >= 0;
    if (!pre_opened && g_prof.on.load(std::memory_order_relaxed)) {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (g_prof.on.load() && g_prof.n < g_prof.cap) rec_slot = g_prof.n++;
    }
    const bool rec = rec_slot >= 0;
    if (rec && !pre_opened) NML_CUDA(cudaEventRecord(g_prof.start[rec_slot], st));
    if (P.pair) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3(grid);
        cfg.blockDim = dim3(threads_for(P.mode == MODE_FPROP ? P.out_mode : OUT_NHWC));
        cfg.dynamicSmemBytes = smem;
        cfg.stream = st;
        cudaLaunchAttribute attr;
        attr.id = cudaLaunchAttributeClusterDimension;
        attr.val.clusterDim.x = 2;
        attr.val.clusterDim.y = 1;
        attr.val.clusterDim.z = 1;
        cfg.attrs = &attr;
        cfg.numAttrs = 1;
        NML_CUDA(cudaLaunchKernelEx(&cfg, kernel_for(P), P));
    } else {
        kernel_for(P)<<<grid, threads_for(P.mode == MODE_FPROP ? P.out_mode : OUT_NHWC), smem, st>>>(P);
    }
    NML_CUDA(cudaGetLastError());
    if (open_slot) *open_slot = rec_slot;
    else if (rec) NML_CUDA(cudaEventRecord(g_prof.stop[rec_slot], st));
    ++g_launches;
    return NML_OK;
}

// ------------------------------------------------------- fprop-like problems --
struct FpropLike {
    const void* a;
    int a_dtype, a_layout, batch, a_c, a_h, a_w;
    const void* w;
    int w_dtype, d0, d1, kh, kw, k_is_dim0, w_direct;
    int gather;  // 0: output pixel o reads input o*s - p + k*d; 1: output pixel o gathers from (o + p - k*d)/s
    int s_h, s_w, p_h, p_w, d_h, d_w;
    void* out;
    int out_dtype, out_layout, out_c, out_h, out_w;
    const void* bias;
    int bias_dtype;
    int math, round_f16;
    // phase-packed gather walk (set by run_fprop_like itself): the real output behind the packed columns
    int shuf_sh, shuf_sw, shuf_c, shuf_oh, shuf_ow;
};

static int run_fprop_like(const FpropLike& f, Bump& ws, cudaStream_t st) {
    MathInfo mi;
    if (!math_info(f.math, &mi)) return NML_ERR_INVALID;
    // A strided gather with very few output channels (input gradient of an RGB stem, image-producing
    // transposed layer) would run one mostly empty 16-column pass per output phase.  All phases are
    // packed into the columns instead: one unit-stride pass over the input with stride_h*stride_w*C
    // columns, whose epilogue scatters each row to its stride_h x stride_w block of output pixels.
    if (f.gather && f.k_is_dim0 && !f.shuf_sh && f.d_h == 1 && f.d_w == 1 && f.s_h * f.s_w > 1 &&
        f.s_h * f.s_w * f.d1 <= 16 && f.out_layout == NML_NHWC && mi.enc == ENC_F16 && f.d1 == f.out_c &&
        tune().shuffle) {
        const int C = f.d1, Kc = f.d0;
        int dh_min = 1 << 20, dh_max = -(1 << 20), dw_min = 1 << 20, dw_max = -(1 << 20);
        for (int ph = 0; ph < f.s_h; ++ph)
            for (int kh = 0; kh < f.kh; ++kh) {
                const int nh = ph + f.p_h - kh;
                if (((nh % f.s_h) + f.s_h) % f.s_h != 0) continue;
                const int dh = (nh >= 0) ? nh / f.s_h : -((-nh) / f.s_h);
                dh_min = std::min(dh_min, dh);
                dh_max = std::max(dh_max, dh);
            }
        for (int pw = 0; pw < f.s_w; ++pw)
            for (int kw = 0; kw < f.kw; ++kw) {
                const int nw = pw + f.p_w - kw;
                if (((nw % f.s_w) + f.s_w) % f.s_w != 0) continue;
                const int dw = (nw >= 0) ? nw / f.s_w : -((-nw) / f.s_w);
                dw_min = std::min(dw_min, dw);
                dw_max = std::max(dw_max, dw);
            }
        if (dh_min <= dh_max && dw_min <= dw_max && (dh_max - dh_min + 1) * (dw_max - dw_min + 1) <= kMaxTaps) {
            const int khp = dh_max - dh_min + 1, kwp = dw_max - dw_min + 1;
            const int np = f.s_h * f.s_w * C;
            __half* wp = static_cast<__half*>(ws.take(static_cast<size_t>(np) * Kc * khp * kwp * sizeof(__half)));
            float* bp = f.bias ? static_cast<float*>(ws.take(sizeof(float) * np)) : nullptr;
            if (!ws.dry) {
                if (!ws.fits()) return NML_ERR_WORKSPACE;
                const int total = np * Kc * khp * kwp;
                const int blocks = std::min(ceil_div(total, 256), 148 * 8);
#define NML_PACK(TW, TB)                                                                                            \
    pack_phase_weights_kernel<TW, TB><<<blocks, 256, 0, st>>>(static_cast<const TW*>(f.w), wp,                      \
                                                              static_cast<const TB*>(f.bias), bp, Kc, C, f.kh, f.kw, \
                                                              f.s_h, f.s_w, f.p_h, f.p_w, khp, kwp, dh_min, dw_min)
                if (f.w_dtype == NML_F32) {
                    if (f.bias_dtype == NML_F16) NML_PACK(float, __half); else NML_PACK(float, float);
                } else {
                    if (f.bias_dtype == NML_F16) NML_PACK(__half, __half); else NML_PACK(__half, float);
                }
#undef NML_PACK
                ++g_launches;
                NML_CUDA(cudaGetLastError());
            }
            FpropLike f2 = f;
            f2.w = wp; f2.w_dtype = NML_F16; f2.d0 = np; f2.d1 = Kc; f2.kh = khp; f2.kw = kwp; f2.k_is_dim0 = 0;
            f2.w_direct = 0; f2.gather = 0; f2.s_h = f2.s_w = 1; f2.p_h = -dh_min; f2.p_w = -dw_min;
            f2.out_c = np; f2.out_h = ceil_div(f.out_h, f.s_h); f2.out_w = ceil_div(f.out_w, f.s_w);
            f2.bias = bp; f2.bias_dtype = NML_F32;
            f2.shuf_sh = f.s_h; f2.shuf_sw = f.s_w; f2.shuf_c = C; f2.shuf_oh = f.out_h; f2.shuf_ow = f.out_w;
            return run_fprop_like(f2, ws, st);
        }
    }
    const int T = f.kh * f.kw;
    const int K = f.k_is_dim0 ? f.d0 : f.d1;
    const int N = f.k_is_dim0 ? f.d1 : f.d0;
    if (K != f.a_c || N != f.out_c) return NML_ERR_INVALID;
    if (T > kMaxTaps || f.s_h * f.s_w > kMaxPhases) return NML_ERR_UNSUPPORTED;
    if (f.batch <= 0 || f.a_c <= 0 || f.a_h <= 0 || f.a_w <= 0 || f.out_c <= 0 || f.out_h <= 0 || f.out_w <= 0)
        return NML_ERR_INVALID;

    DeviceState* ds = ws.ds;
    if (!ws.dry && !ds) {
        int rc = device_state(&ds);
        if (rc) return rc;
    }
    // Few input channels (RGB stems): one K slice per kernel ROW, holding (kw, c) for 8 taps, read
    // as overlapping 8-pixel windows of a padded 8-channel image -- instead of one mostly empty
    // 64-channel slice per tap.
    const bool window = !f.gather && !f.k_is_dim0 && T > 1 && window_eligible(f.a_c, f.kw, f.d_w, mi.enc);
    WindowImage wimg = {nullptr, 0, 0};
    // activation operand
    const void* a_planes[2] = {nullptr, nullptr};
    int Cp = 0;
    int rc;
    if (window)
        rc = prepare_window(f.a, f.a_dtype, f.a_layout, f.batch, f.a_c, f.a_h, f.a_w, f.p_h, f.p_w, f.s_w, f.out_w, ws, st,
                            &wimg);
    else
        rc = prepare_activation(f.a, f.a_dtype, f.a_layout, f.batch, f.a_c, f.a_h, f.a_w, mi, ws, st, a_planes, &Cp,
                                nullptr);
    if (rc) return rc;
    if (window) a_planes[0] = wimg.ptr;
    // weight operand
    const int c_blocks = window ? 1 : ceil_div(K, mi.kb);
    const int kp = c_blocks * mi.kb;
    const int align = 16 / mi.es;
    bool direct_w = !window && f.w_direct && T == 1 && mi.enc == ENC_F16 && f.w_dtype == NML_F16 &&
                    ((f.k_is_dim0 ? N : K) % align == 0);
    const void* w_planes[2] = {f.w, nullptr};
    int b_mn_major = 0;
    if (window) {
        void* p0 = ws.take(static_cast<size_t>(N) * f.kh * 64 * 2);
        w_planes[0] = p0;
        if (!ws.dry) {
            if (!ws.fits()) return NML_ERR_WORKSPACE;
            int blocks = std::min(ceil_div(N * f.kh * 64, 256), 148 * 8);
            if (f.w_dtype == NML_F32)
                { repack_weight_c8_kernel<float><<<blocks, 256, 0, st>>>(static_cast<const float*>(f.w), static_cast<__half*>(p0), N, K, f.kh, f.kw); ++g_launches; }
            else
                { repack_weight_c8_kernel<__half><<<blocks, 256, 0, st>>>(static_cast<const __half*>(f.w), static_cast<__half*>(p0), N, K, f.kh, f.kw); ++g_launches; }
            NML_CUDA(cudaGetLastError());
        }
    } else if (direct_w) {
        b_mn_major = f.k_is_dim0 ? 1 : 0;
    } else {
        size_t bytes = static_cast<size_t>(N) * T * kp * mi.es;
        void* p0 = ws.take(bytes);
        void* p1 = (mi.planes == 2) ? ws.take(bytes) : nullptr;
        w_planes[0] = p0;
        w_planes[1] = p1;
        if (!ws.dry) {
            if (!ws.fits()) return NML_ERR_WORKSPACE;
            // out[n][t][k] = w[...]: a swap of the two inner dimensions of [B][R][Cc] (see repack_weight_*_kernel)
            const int rB = f.k_is_dim0 ? 1 : f.d0, rR = f.k_is_dim0 ? f.d0 : f.d1, rC = f.k_is_dim0 ? f.d1 * T : T;
            if (rB > 65535) return NML_ERR_UNSUPPORTED;
#define NML_REPACK(T)                                                                                                           \
    do {                                                                                                                        \
        if (rC <= 64)                                                                                                           \
            repack_weight_rows_kernel<T><<<dim3(ceil_div(kp, 64), rB), 256, 0, st>>>(static_cast<const T*>(f.w), p0, p1, mi.enc, \
                                                                                     rR, rC, kp);                               \
        else                                                                                                                    \
            repack_weight_tile_kernel<T><<<dim3(ceil_div(rC, 64), ceil_div(kp, 64), rB), 256, 0, st>>>(                          \
                static_cast<const T*>(f.w), p0, p1, mi.enc, rR, rC, kp);                                                         \
    } while (0)
            if (f.w_dtype == NML_F32) NML_REPACK(float); else NML_REPACK(__half);
#undef NML_REPACK
            ++g_launches;
            NML_CUDA(cudaGetLastError());
        }
    }
    // Bias as fp32: the TMA-store epilogues read an fp16 bias as it is (they stage the tile's bias values in
    // shared memory once per column tile anyway); the other epilogues and the finishing pass of a K-split walk
    // take a widened copy, made just before the launch once the plan is known.
    const float* bias32 = static_cast<const float*>(f.bias);
    const bool bias_is_f16 = f.bias && f.bias_dtype == NML_F16;
    float* bias_widened = bias_is_f16 ? static_cast<float*>(ws.take(sizeof(float) * N)) : nullptr;
    if (bias_is_f16) bias32 = bias_widened;
    // Few output pixels under a long K loop (the 2x2 ... 8x8 layers of a U-Net): room for the fp32 partial
    // sums of a K-split walk.
    const size_t out_pixels = static_cast<size_t>(f.batch) * f.out_h * f.out_w;
    const bool may_split = !window && !f.shuf_sh && T >= 4 && out_pixels <= 8192 && 1ll * T * c_blocks >= 32 && tune().fsplit;
    // one fp32 plane per K slice; the bound on the slice count below holds for every plan made further down
    // (tiles >= tiles_lb, at least 4 K iterations per slice)
    int z_cap = 1;
    if (may_split) {
        const long long tiles_lb = 1ll * ((out_pixels + 127) / 128) * ceil_div(N, 256);
        const int sms = ds ? limited(ds->sms) : planning_sms();
        z_cap = static_cast<int>(std::max<long long>(1, std::min<long long>(sms / tiles_lb, 1ll * (mi.planes == 2 ? 3 : 1) * T * c_blocks / 4)));
    }
    float* split_acc = may_split ? static_cast<float*>(ws.take(static_cast<size_t>(z_cap) * out_pixels * N * sizeof(float))) : nullptr;
    if (ws.dry) return NML_OK;
    if (!ws.fits()) return NML_ERR_WORKSPACE;

    KParams P;
    memset(&P, 0, sizeof(P));
    P.mode = MODE_FPROP;
    P.out_mode = (f.out_layout == NML_NCHW && !(f.out_h == 1 && f.out_w == 1)) ? OUT_NCHW : OUT_NHWC;
    P.kind = mi.kind;
    P.passes = (mi.planes == 2) ? 3 : 1;
    P.kb = mi.kb;
    P.c_blocks = c_blocks;
    P.a_mn_major = 0;
    P.b_mn_major = b_mn_major;
    P.batch = f.batch;
    P.n_tiles = ceil_div(N, 256);  // provisional; the tile width is settled once the row tiles are known
    P.bn = static_cast<int>(round_up(ceil_div(N, P.n_tiles), b_mn_major ? 64 : 32));
    P.out = f.out;
    P.bias = bias32;
    P.out_f16 = (f.out_dtype == NML_F16);
    P.round_f16 = f.round_f16;
    P.c_out = N;
    P.shuf_sh = f.shuf_sh;
    P.shuf_sw = f.shuf_sw;
    P.shuf_c = f.shuf_c;
    P.shuf_oh = f.shuf_oh;
    P.shuf_ow = f.shuf_ow;
    P.out_h = f.out_h;
    P.out_w = f.out_w;
    P.ld_out = N;

    // phases and taps
    int n_taps = 0, n_phases = 0;
    if (window) {
        Phase& ph = P.phases[0];
        ph.ph = ph.pw = 0;
        ph.hq = f.out_h;
        ph.wq = f.out_w;
        ph.tap_begin = 0;
        for (int kh = 0; kh < f.kh; ++kh) {  // the padding is physical: offsets start at 0
            Tap& t = P.taps[n_taps++];
            t.dh = static_cast<short>(kh * f.d_h);
            t.dw = 0;
            t.wk = kh * 64;
        }
        ph.tap_count = static_cast<short>(n_taps);
        n_phases = 1;
        P.a_stride_h = f.s_h;  // rows of the padded image
        P.a_stride_w = 1;      // the window dimension is already indexed by output column
        P.out_stride_h = P.out_stride_w = 1;
    } else if (!f.gather) {
        Phase& ph = P.phases[0];
        ph.ph = ph.pw = 0;
        ph.hq = f.out_h;
        ph.wq = f.out_w;
        ph.tap_begin = 0;
        for (int kh = 0; kh < f.kh; ++kh)
            for (int kw = 0; kw < f.kw; ++kw) {
                Tap& t = P.taps[n_taps++];
                t.dh = static_cast<short>(kh * f.d_h - f.p_h);
                t.dw = static_cast<short>(kw * f.d_w - f.p_w);
                t.wk = direct_w ? 0 : (kh * f.kw + kw) * kp;
            }
        ph.tap_count = static_cast<short>(n_taps);
        n_phases = 1;
        P.a_stride_h = f.s_h;
        P.a_stride_w = f.s_w;
        P.out_stride_h = P.out_stride_w = 1;
    } else {
        for (int ph_ = 0; ph_ < f.s_h; ++ph_)
            for (int pw_ = 0; pw_ < f.s_w; ++pw_) {
                if (ph_ >= f.out_h || pw_ >= f.out_w) continue;
                Phase& ph = P.phases[n_phases++];
                ph.ph = static_cast<short>(ph_);
                ph.pw = static_cast<short>(pw_);
                ph.hq = ceil_div(f.out_h - ph_, f.s_h);
                ph.wq = ceil_div(f.out_w - pw_, f.s_w);
                ph.tap_begin = static_cast<short>(n_taps);
                for (int kh = 0; kh < f.kh; ++kh) {
                    int nh = ph_ + f.p_h - kh * f.d_h;
                    if (((nh % f.s_h) + f.s_h) % f.s_h != 0) continue;
                    for (int kw = 0; kw < f.kw; ++kw) {
                        int nw = pw_ + f.p_w - kw * f.d_w;
                        if (((nw % f.s_w) + f.s_w) % f.s_w != 0) continue;
                        Tap& t = P.taps[n_taps++];
                        t.dh = static_cast<short>(nh / f.s_h);
                        t.dw = static_cast<short>(nw / f.s_w);
                        t.wk = direct_w ? 0 : (kh * f.kw + kw) * kp;
                    }
                }
                ph.tap_count = static_cast<short>(n_taps - ph.tap_begin);
            }
        P.a_stride_h = P.a_stride_w = 1;
        P.out_stride_h = f.s_h;
        P.out_stride_w = f.s_w;
    }
    P.n_phases = n_phases;
    // M-tile box from the largest phase grid
    const int esw = (f.gather || window) ? 1 : f.s_w, esh = f.gather ? 1 : f.s_h;
    choose_box(7, P.phases[0].wq, P.phases[0].hq, f.batch, esw, esh, &P.wb_log2, &P.hb_log2, &P.nb_log2,
               (P.out_mode == OUT_NCHW && !f.gather) ? 5 : 0);
    bool patch_resident = false;
    // Patch walk: unit-stride walks with several taps load one haloed patch per channel block instead of
    // one box per tap (8 x 16 pixel tiles of a single image).  Taken when the fixed tile shape does not
    // waste much more of the tile than the free-form box does.  Every phase of a gather walk has its own
    // taps and patch origin; the box is sized for the widest phase.
    {
        const int mode = tune().patch;
        int range_w = 0, range_h = 0;
        bool every_phase_has_taps = true;
        for (int p = 0; p < n_phases; ++p) {
            Phase& ph = P.phases[p];
            if (ph.tap_count == 0) {
                every_phase_has_taps = false;
                continue;
            }
            int dw_min = 0, dw_max = 0, dh_min = 0, dh_max = 0;
            for (int t = 0; t < ph.tap_count; ++t) {
                const Tap& tp = P.taps[ph.tap_begin + t];
                dw_min = t ? std::min<int>(dw_min, tp.dw) : tp.dw;
                dw_max = t ? std::max<int>(dw_max, tp.dw) : tp.dw;
                dh_min = t ? std::min<int>(dh_min, tp.dh) : tp.dh;
                dh_max = t ? std::max<int>(dh_max, tp.dh) : tp.dh;
            }
            ph.org_w = static_cast<short>(dw_min);
            ph.org_h = static_cast<short>(dh_min);
            range_w = std::max(range_w, dw_max - dw_min);
            range_h = std::max(range_h, dh_max - dh_min);
        }
        // (a row stride of the walk only stretches the patch: consecutive output rows are esh patch rows apart)
        const int pw_ = 8 + range_w, ph_ = 15 * esh + range_h + 1;
        const int wq = P.phases[0].wq, hq = P.phases[0].hq;
        const double eff_patch = static_cast<double>(wq) * hq / (1.0 * round_up(wq, 8) * round_up(hq, 16));
        const double eff_box = static_cast<double>(wq) * hq * f.batch /
                               (1.0 * round_up(wq, 1 << P.wb_log2) * round_up(hq, 1 << P.hb_log2) * round_up(f.batch, 1 << P.nb_log2));
        const bool can = every_phase_has_taps && n_taps >= 2 && esw == 1 && pw_ <= 256 && ph_ <= 256 &&
                         pw_ * ph_ * 128 <= 48 * 1024;
        // B stays resident when every slice fits beside two patch buffers and the smallest epilogue staging;
        // streaming B tap by tap pays only for the 3xTF32 split (a barrier round trip per 4 short MMAs otherwise)
        const int bn_res = (N <= 16 && !b_mn_major) ? 16 : static_cast<int>(round_up(N, 32));
        const long long res_need = 1ll * c_blocks * n_taps * bn_res * 128 + 2 * round_up(pw_ * ph_ * 128, 1024);
        const bool res_ok = P.passes == 1 && N <= 256 &&
                            res_need <= 232448 - (1024 + 256 + kBiasTileBytes) - 4 * kStagingBufBytes;
        const bool streamed_ok = N <= 128 && (P.passes == 3 || mode >= 3);
        if (can && mode && (mode == 2 || (eff_patch >= 0.8 * eff_box && (res_ok || streamed_ok)))) {
            patch_resident = res_ok;
            P.patch = 1;
            P.patch_w = pw_;
            P.patch_h = ph_;
            P.patch_bytes = static_cast<int>(round_up(pw_ * ph_ * 128, 1024));
            for (int p = 0; p < n_phases; ++p)
                for (int t = 0; t < P.phases[p].tap_count; ++t) {
                    Tap& tp = P.taps[P.phases[p].tap_begin + t];
                    tp.aoff = ((tp.dh - P.phases[p].org_h) * pw_ + (tp.dw - P.phases[p].org_w)) * 128 / 16;
                }
            P.n_taps = n_taps;
            P.wb_log2 = 3;
            P.hb_log2 = 4;
            P.nb_log2 = 0;
        }
    }
    // Tile width: 256 columns run the tensor pipe best, but when that leaves SMs idle (few row tiles,
    // narrow N) a narrower tile wins.  Cost per column relative to a 256-wide tile, measured on B200:
    // 128 -> 1.28, 64 -> 2.24; the makespan is rounds x width x cost.
    {
        long long m_tiles_all = 0;
        for (int p = 0; p < n_phases; ++p)
            m_tiles_all += 1ll * ceil_div(P.phases[p].wq, 1 << P.wb_log2) * ceil_div(P.phases[p].hq, 1 << P.hb_log2) *
                           ceil_div(f.batch, 1 << P.nb_log2);
        const int forced = (P.patch && patch_resident) ? ((N <= 16 && !b_mn_major) ? 16 : static_cast<int>(round_up(N, 32)))
                                                       : tune().bn;
        const int cand[4] = {256, 128, 64, forced};
        const double cost[3] = {1.0, 1.28, 2.24};
        double best = -1;
        for (int i = 0; i < 4; ++i) {
            if (forced ? i != 3 : i == 3) continue;
            int nt = ceil_div(N, cand[i]);
            int bn = static_cast<int>(round_up(ceil_div(N, nt), b_mn_major ? 64 : (forced == 16 ? 16 : 32)));
            if (bn > 256) continue;
            double rounds = static_cast<double>(ceil_div(static_cast<int>(std::min<long long>(m_tiles_all * nt, 1 << 30)), limited(ds->sms)));
            double t = rounds * bn * (bn > 128 ? cost[0] : bn > 64 ? cost[1] : cost[2]);
            if (best < 0 || t < best * 0.97) {  // prefer the wider tile unless the gain is clear
                best = t;
                P.n_tiles = nt;
                P.bn = bn;
            }
        }
    }
    // Row-major output through TMA stores when the geometry allows: the box is the 32 consecutive tile
    // rows one epilogue warp owns (a sub-box of the tile's pixel box), 128 bytes of columns wide.
    if (P.out_mode == OUT_NHWC && tune().tmastore) {
        const int esz = P.out_f16 ? 2 : 4;
        const int cpi = 128 / esz;
        if (P.bn % cpi == 0 && (static_cast<size_t>(N) * esz) % 16 == 0 && (reinterpret_cast<uintptr_t>(f.out) & 15) == 0) {
            const int wbx = 1 << P.wb_log2, hbx = 1 << P.hb_log2;
            const int bw = std::min(wbx, 32), bh = std::min(hbx, 32 / bw), bnn = 32 / (bw * bh);
            uint64_t cd[4] = {static_cast<uint64_t>(N), static_cast<uint64_t>(f.out_w), static_cast<uint64_t>(f.out_h),
                              static_cast<uint64_t>(f.batch)};
            uint32_t cb[4] = {static_cast<uint32_t>(cpi), static_cast<uint32_t>(bw * P.out_stride_w),
                              static_cast<uint32_t>(bh * P.out_stride_h), static_cast<uint32_t>(bnn)};
            uint32_t ce[4] = {1, static_cast<uint32_t>(P.out_stride_w), static_cast<uint32_t>(P.out_stride_h), 1};
            if (cb[1] <= 256 && cb[2] <= 256 && encode_map(&P.tmC, f.out, esz, 4, cd, cb, ce, SWZ_128B) == NML_OK)
                P.out_mode = OUT_NHWC_TMA;
        }
    }
    // Channel-major (NCHW) output through TMA stores: box = the (w, h) sub-box of the warp's 32 pixels x 64 fp16 / 32 fp32 channels, staged channel-major.  Needs
    // unit output stride (TMA cannot stride the innermost dimension) and 16-byte aligned rows.
    if (P.out_mode == OUT_NCHW && tune().tmastore && P.out_stride_w == 1 && P.out_stride_h == 1) {
        const int esz = P.out_f16 ? 2 : 4;
        const int cpi = 128 / esz;
        const int wbx = 1 << P.wb_log2, hbx = 1 << P.hb_log2;
        const int bw = std::min(wbx, 32), bh = std::min(hbx, 32 / bw), bnn = 32 / (bw * bh);
        if (P.bn % cpi == 0 && (bw * esz) % 16 == 0 && (static_cast<size_t>(f.out_w) * esz) % 16 == 0 &&
            (reinterpret_cast<uintptr_t>(f.out) & 15) == 0) {
            uint64_t cd[4] = {static_cast<uint64_t>(f.out_w), static_cast<uint64_t>(f.out_h), static_cast<uint64_t>(N),
                              static_cast<uint64_t>(f.batch)};
            uint32_t cb[4] = {static_cast<uint32_t>(bw), static_cast<uint32_t>(bh), static_cast<uint32_t>(cpi),
                              static_cast<uint32_t>(bnn)};
            uint32_t ce[4] = {1, 1, 1, 1};
            if (encode_map(&P.tmC, f.out, esz, 4, cd, cb, ce, SWZ_NONE) == NML_OK) {
                P.out_mode = OUT_NCHW_TMA;
                int l = 0;
                while ((1 << l) < bw) ++l;
                P.cm_bw_log2 = l;
                l = 0;
                while ((1 << l) < bh) ++l;
                P.cm_bh_log2 = l;
            }
        }
    }
    // Pairs of CTAs (cta_group::2) for 256-wide tiles of problems large enough to fill the pairs: a
    // tile id then names two consecutive row tiles of one phase.
    // (short K loops are epilogue-bound, where pairing only halves the number of independent tiles)
    const int k_iters_min = P.passes * P.c_blocks * std::max<int>(1, P.phases[0].tap_count);
    // (a problem with so few tiles that half the SMs would idle is K-split instead, see below)
    long long tiles_single = 0;
    for (int p = 0; p < n_phases; ++p)
        tiles_single += 1ll * ceil_div(P.phases[p].wq, 1 << P.wb_log2) * ceil_div(P.phases[p].hq, 1 << P.hb_log2) *
                        ceil_div(f.batch, 1 << P.nb_log2) * P.n_tiles;
    const bool will_split = may_split && !P.patch && tiles_single * 2 <= limited(ds->sms) && k_iters_min >= 8;
    // 128-column tiles pair up too (two K slices per stage, see launch_kernel) where every phase has a K loop
    // of at least four slices and the tiles fill most of the GPU: measured 5-15 % on such layers, a loss on
    // the short phases of strided gathers and on few-tile problems.
    int k_iters_all = k_iters_min;
    for (int p = 0; p < n_phases; ++p)
        if (P.phases[p].tap_count > 0) k_iters_all = std::min(k_iters_all, P.passes * P.c_blocks * P.phases[p].tap_count);
    const bool pair_width = P.bn == 256 || (tune().pair128 && P.bn == 128 && k_iters_all >= 4 && tiles_single * 4 >= 3ll * limited(ds->sms));
    P.pair = (tune().pair && !P.patch && !will_split && pair_width && (!b_mn_major || N % mi.kb == 0) && k_iters_min >= 4 &&
              (P.out_mode == OUT_NHWC_TMA || P.out_mode == OUT_NCHW_TMA || P.out_mode == OUT_NCHW) && limited(ds->sms) >= 2) ? 1 : 0;
    int tiles = 0;
    for (int p = 0; p < n_phases; ++p) {
        Phase& ph = P.phases[p];
        ph.tiles_w = ceil_div(ph.wq, 1 << P.wb_log2);
        ph.tiles_h = ceil_div(ph.hq, 1 << P.hb_log2);
        ph.tile_begin = tiles;
        int m_tiles = ph.tiles_w * ph.tiles_h * ceil_div(f.batch, 1 << P.nb_log2);
        tiles += (P.pair ? ceil_div(m_tiles, 2) : m_tiles) * P.n_tiles;
    }
    P.num_tiles = tiles;
    P.base_tiles = tiles;
    {   // division by multiplication in the kernels' tile decode: exact while tile index x divisor < 2^40
        const unsigned long long one40 = 1ull << 40;
        long long dmax = P.n_tiles;
        P.mul_nt = one40 / static_cast<unsigned long long>(P.n_tiles) + 1;
        for (int p = 0; p < n_phases; ++p) {
            Phase& ph = P.phases[p];
            ph.mul_w = one40 / static_cast<unsigned long long>(std::max(1, ph.tiles_w)) + 1;
            ph.mul_h = one40 / static_cast<unsigned long long>(std::max(1, ph.tiles_h)) + 1;
            dmax = std::max<long long>(dmax, std::max(ph.tiles_w, ph.tiles_h));
        }
        // (a pair doubles the row-tile index before it is divided)
        P.fastdiv = (2ll * tiles < (1ll << 23) && 2ll * tiles * dmax < (1ll << 40)) ? 1 : 0;
    }
    P.fsplit = 1;
    if (may_split && !P.pair && !P.patch && tiles * 2 <= limited(ds->sms)) {
        int k_min = k_iters_min;
        for (int p = 0; p < n_phases; ++p)
            if (P.phases[p].tap_count > 0) k_min = std::min(k_min, P.passes * P.c_blocks * P.phases[p].tap_count);
        const int z = std::min(z_cap, std::min(limited(ds->sms) / tiles, k_min / 4));  // at least 4 K iterations per slice
        if (z >= 2) {
            P.fsplit = z;
            P.num_tiles = tiles * z;
            // slice z stores into plane z of the scratch; the finishing pass adds the planes in order and
            // applies bias, rounding, cast and layout
            P.plane_elems = out_pixels * N;
            P.out = split_acc;
            P.out_mode = OUT_NHWC;
            P.out_f16 = 0;
            P.round_f16 = 0;
            P.bias = nullptr;
            P.ld_out = N;
        }
    }

    // tensor maps
    for (int pl = 0; pl < mi.planes; ++pl) {
        uint64_t adims[4] = {static_cast<uint64_t>(Cp), static_cast<uint64_t>(f.a_w), static_cast<uint64_t>(f.a_h),
                             static_cast<uint64_t>(f.batch)};
        uint32_t abox[4] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>((1 << P.wb_log2) * esw),
                            static_cast<uint32_t>((1 << P.hb_log2) * esh), static_cast<uint32_t>(1 << P.nb_log2)};
        uint32_t aes[4] = {1, static_cast<uint32_t>(esw), static_cast<uint32_t>(esh), 1};
        if (P.patch) {  // contiguous rows: the row stride is applied by the MMA descriptors
            abox[1] = static_cast<uint32_t>(P.patch_w);
            abox[2] = static_cast<uint32_t>(P.patch_h);
            abox[3] = 1;
            aes[1] = aes[2] = 1;
        }
        if (window) {
            // dims: (64 elements = 8 pixels x 8 channels, output column, padded row, image); consecutive
            // output columns start s_w pixels apart, so the windows overlap
            uint64_t wd[4] = {64, static_cast<uint64_t>(f.out_w), static_cast<uint64_t>(wimg.hp), static_cast<uint64_t>(f.batch)};
            uint64_t wstr[3] = {static_cast<uint64_t>(f.s_w) * 16, static_cast<uint64_t>(wimg.wp) * 16,
                                static_cast<uint64_t>(wimg.hp) * wimg.wp * 16};
            rc = encode_map(&P.tmA[pl], a_planes[pl], 2, 4, wd, abox, aes, SWZ_128B, wstr);
        } else {
            rc = encode_map(&P.tmA[pl], a_planes[pl], mi.es, 4, adims, abox, aes, SWZ_128B);
        }
        if (rc) return rc;
        uint32_t one[2] = {1, 1};
        if (!b_mn_major) {
            uint64_t bdims[2] = {static_cast<uint64_t>(direct_w ? K : (window ? f.kh * 64 : T * kp)), static_cast<uint64_t>(N)};
            uint32_t bbox[2] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>(P.pair ? P.bn / 2 : P.bn)};
            rc = encode_map(&P.tmB[pl], w_planes[pl], mi.es, 2, bdims, bbox, one, SWZ_128B);
        } else if (N % mi.kb == 0) {
            // one box per stage: the outermost dimension walks the 128-byte column groups
            P.b_grouped = 1;
            uint64_t bdims[3] = {static_cast<uint64_t>(mi.kb), static_cast<uint64_t>(K), static_cast<uint64_t>(N / mi.kb)};
            uint64_t bstr[2] = {static_cast<uint64_t>(N) * mi.es, static_cast<uint64_t>(mi.kb) * mi.es};
            uint32_t bbox[3] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>(mi.kb),
                                static_cast<uint32_t>((P.pair ? P.bn / 2 : P.bn) / mi.kb)};
            uint32_t one3[3] = {1, 1, 1};
            rc = encode_map(&P.tmB[pl], w_planes[pl], mi.es, 3, bdims, bbox, one3, SWZ_128B, bstr);
        } else {
            uint64_t bdims[2] = {static_cast<uint64_t>(N), static_cast<uint64_t>(K)};
            uint32_t bbox[2] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>(mi.kb)};
            rc = encode_map(&P.tmB[pl], w_planes[pl], mi.es, 2, bdims, bbox, one, SWZ_128B);
        }
        if (rc) return rc;
    }
    if (g_dbg_short_a_box) {
        // nml_debug_stalled_linear_forward only: A boxes half as tall as the kernel expects, so no stage
        // ever receives all its bytes and the bounded waits run out
        uint64_t adims[4] = {static_cast<uint64_t>(Cp), static_cast<uint64_t>(f.a_w), static_cast<uint64_t>(f.a_h),
                             static_cast<uint64_t>(f.batch)};
        uint32_t abox[4] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>((1 << P.wb_log2) / 2), 1, 1};
        uint32_t aes[4] = {1, 1, 1, 1};
        rc = encode_map(&P.tmA[0], a_planes[0], mi.es, 4, adims, abox, aes, SWZ_128B);
        if (rc) return rc;
    }
    if (bias_is_f16) {
        if (NML_IS_TMA_OUT(P.out_mode) && P.fsplit <= 1 && P.bias != nullptr) {
            P.bias = static_cast<const float*>(f.bias);  // read as __half by the kernel
            P.bias_f16 = 1;
        } else {
            to_float_kernel<__half><<<ceil_div(N, 256), 256, 0, st>>>(static_cast<const __half*>(f.bias), bias_widened, N);
            ++g_launches;
        }
    }
    int slot = -1;
    rc = launch_kernel(P, ds, st, &slot);
    if (rc) return rc;
    if (P.fsplit <= 1) return profile_stop(slot, st);
    {
        const size_t total = out_pixels * N;
        const int blocks = static_cast<int>(std::min<size_t>((total + 255) / 256, 148 * 8));
        const int nchw = (f.out_layout == NML_NCHW && !(f.out_h == 1 && f.out_w == 1)) ? 1 : 0;
        if (f.out_dtype == NML_F16)
            { finish_rows_kernel<__half><<<blocks, 256, 0, st>>>(split_acc, P.fsplit, bias32, static_cast<__half*>(f.out), out_pixels, N,
                                                              f.out_h * f.out_w, nchw, 0); ++g_launches; }
        else
            { finish_rows_kernel<float><<<blocks, 256, 0, st>>>(split_acc, P.fsplit, bias32, static_cast<float*>(f.out), out_pixels, N,
                                                             f.out_h * f.out_w, nchw, f.round_f16); ++g_launches; }
        NML_CUDA(cudaGetLastError());
    }
    return profile_stop(slot, st);
}

// ------------------------------------------------------- wgrad-like problems --
struct WgradLike {
    const void* patch;  // tensor the (tap-shifted, strided) patches are cut from
    int patch_c, patch_h, patch_w;
    const void* plain;  // tensor indexed by the pixel itself
    int plain_c, plain_h, plain_w;
    int dtype, layout, batch;
    int kh, kw, s_h, s_w, p_h, p_w, d_h, d_w;
    float* dw;  // [plain_c][patch_c][kh*kw]
    float* colsum;
    int colsum_of_patch;
    int math;
};

static int run_wgrad_like(const WgradLike& g, Bump& ws, cudaStream_t st) {
    MathInfo mi;
    if (!math_info(g.math, &mi)) return NML_ERR_INVALID;
    const int T = g.kh * g.kw;
    if (T > kMaxTaps) return NML_ERR_UNSUPPORTED;
    if (g.batch <= 0 || g.patch_c <= 0 || g.plain_c <= 0 || g.patch_h <= 0 || g.patch_w <= 0 || g.plain_h <= 0 ||
        g.plain_w <= 0)
        return NML_ERR_INVALID;
    DeviceState* ds = nullptr;
    if (!ws.dry) {
        int rc = device_state(&ds);
        if (rc) return rc;
    }
    const int sms = ds ? limited(ds->sms) : planning_sms();
    const void* pa[2] = {nullptr, nullptr};
    const void* pb[2];
    int cpa = 0, cpb = 0;
    // Few-channel layer input (RGB stems): patches come as 8-pixel windows of the padded 8-channel image,
    // one kernel row per tap, (kw, c) packed in the 64 patch columns.
    const bool window = T > 1 && window_eligible(g.patch_c, g.kw, g.d_w, mi.enc);
    WindowImage wimg = {nullptr, 0, 0};
    int rc;
    if (window) {
        rc = prepare_window(g.patch, g.dtype, g.layout, g.batch, g.patch_c, g.patch_h, g.patch_w, g.p_h, g.p_w, g.s_w,
                            g.plain_w, ws, st, &wimg, g.colsum_of_patch ? g.colsum : nullptr);
        pa[0] = wimg.ptr;
        cpa = 8;
    } else {
        rc = prepare_activation(g.patch, g.dtype, g.layout, g.batch, g.patch_c, g.patch_h, g.patch_w, mi, ws, st, pa,
                                &cpa, g.colsum_of_patch ? g.colsum : nullptr);
    }
    if (rc) return rc;
    rc = prepare_activation(g.plain, g.dtype, g.layout, g.batch, g.plain_c, g.plain_h, g.plain_w, mi, ws, st, pb, &cpb,
                            g.colsum_of_patch ? nullptr : g.colsum);
    if (rc) return rc;

    KParams P;
    memset(&P, 0, sizeof(P));
    P.mode = MODE_WGRAD;
    P.kind = mi.kind;
    P.passes = (mi.planes == 2) ? 3 : 1;
    P.kb = mi.kb;
    P.a_mn_major = 1;
    P.b_mn_major = 1;
    P.batch = g.batch;
    P.c_blocks = window ? 1 : ceil_div(g.patch_c, mi.kb);
    P.groups_total = (window ? g.kh : T) * P.c_blocks;
    P.c_patch = g.patch_c;
    P.c_plain = g.plain_c;
    P.n_taps = window ? g.kh : T;
    P.kw_pack = window ? 1 : 0;
    P.kw_count = g.kw;
    P.n_tiles = ceil_div(g.plain_c, 256);
    P.bn = static_cast<int>(round_up(ceil_div(g.plain_c, P.n_tiles), 64));
    P.c_out = g.plain_c;
    P.a_stride_h = g.s_h;
    P.a_stride_w = window ? 1 : g.s_w;
    P.out_stride_h = P.out_stride_w = 1;
    if (window) {
        for (int kh = 0; kh < g.kh; ++kh) {
            Tap& t = P.taps[kh];
            t.dh = static_cast<short>(kh * g.d_h);
            t.dw = 0;
            t.wk = kh;
        }
    } else
    for (int kh = 0; kh < g.kh; ++kh)
        for (int kw = 0; kw < g.kw; ++kw) {
            Tap& t = P.taps[kh * g.kw + kw];
            t.dh = static_cast<short>(kh * g.d_h - g.p_h);
            t.dw = static_cast<short>(kw * g.d_w - g.p_w);
            t.wk = kh * g.kw + kw;
        }
    const int bits = (mi.kb == 64) ? 6 : 5;
    choose_box(bits, g.plain_w, g.plain_h, g.batch, window ? 1 : g.s_w, g.s_h, &P.wb_log2, &P.hb_log2, &P.nb_log2);
    // Patch walk: one 64-channel group per tap, unit column stride, few enough row tiles for TMEM, 8 x 8 pixel
    // K blocks that do not waste much of the image, the other tensor fetched as grouped boxes.
    {
        const int groups = P.groups_total;
        const int mt = ceil_div(groups, 2);
        int dw_min = 0, dw_max = 0, dh_min = 0, dh_max = 0;
        for (int t = 0; t < P.n_taps; ++t) {
            dw_min = t ? std::min<int>(dw_min, P.taps[t].dw) : P.taps[t].dw;
            dw_max = t ? std::max<int>(dw_max, P.taps[t].dw) : P.taps[t].dw;
            dh_min = t ? std::min<int>(dh_min, P.taps[t].dh) : P.taps[t].dh;
            dh_max = t ? std::max<int>(dh_max, P.taps[t].dh) : P.taps[t].dh;
        }
        const int pw_ = 8 + dw_max - dw_min, ph_ = 7 * g.s_h + dh_max - dh_min + 1;
        const int bn_w = std::min(256, (512 / std::max(mt, 1)) / 64 * 64);
        const double eff = static_cast<double>(g.plain_w) * g.plain_h / (1.0 * round_up(g.plain_w, 8) * round_up(g.plain_h, 8));
        if (tune().wpatch && mi.enc == ENC_F16 && P.c_blocks == 1 && groups >= 2 && mt <= 8 &&
            (window || g.s_w == 1) && bn_w >= 64 && cpb % 64 == 0 && pw_ <= 256 && ph_ <= 256 &&
            pw_ * ph_ * 128 <= 40 * 1024 && eff >= 0.7) {
            P.wpatch = 1;
            P.w_mtiles = mt;
            P.bn = std::min(bn_w, static_cast<int>(round_up(g.plain_c, 64)));
            P.n_tiles = ceil_div(g.plain_c, P.bn);
            P.patch_w = pw_;
            P.patch_h = ph_;
            P.patch_bytes = static_cast<int>(round_up(pw_ * ph_ * 128, 1024));
            P.phases[0].org_w = static_cast<short>(dw_min);
            P.phases[0].org_h = static_cast<short>(dh_min);
            for (int t = 0; t < P.n_taps; ++t)
                P.taps[t].aoff = ((P.taps[t].dh - dh_min) * pw_ + (P.taps[t].dw - dw_min)) * 128 / 16;
            P.wb_log2 = 3;
            P.hb_log2 = 3;
            P.nb_log2 = 0;
        }
    }
    P.ktiles_w = ceil_div(g.plain_w, 1 << P.wb_log2);
    P.ktiles_h = ceil_div(g.plain_h, 1 << P.hb_log2);
    P.kblocks_total = P.ktiles_w * P.ktiles_h * ceil_div(g.batch, 1 << P.nb_log2);
    // CTA pairs when both operands come as grouped boxes and the tile is 256 columns wide
    const int G_ = kTileM / mi.kb;
    const bool a_grp = !window && (cpa % mi.kb == 0) && (P.c_blocks % G_ == 0);
    const bool b_grp = (cpb % mi.kb == 0);
    P.pair = (tune().pair && !P.wpatch && P.bn == 256 && a_grp && b_grp && sms >= 2) ? 1 : 0;
    const int m_tiles = P.wpatch ? 1 : P.pair ? ceil_div(ceil_div(P.groups_total * mi.kb, kTileM), 2) : ceil_div(P.groups_total * mi.kb, kTileM);
    const int mn_tiles = m_tiles * P.n_tiles;
    // Split K so that the CTAs finish together: the makespan is (rounds of tiles per CTA) x (K
    // blocks per slice, plus a few blocks' worth of prologue / epilogue per tile).  Pick the split
    // that minimises it; ties go to the smaller split (fewer atomics).
    int split = 1;
    {
        // Costs in microseconds: a K block of a 256-wide tile keeps the tensor pipe busy for ~0.27 us (four
        // 128-clock MMAs); more than one slice adds the second-stage reduction, which writes and re-reads one
        // plane of dW per slice and then writes dW (~5 TB/s), plus its launch.
        const double block_us = 0.27 * P.bn / 256.0 * P.passes;
        const double dw_bytes = 4.0 * g.plain_c * g.patch_c * T;
        double best = -1;
        const int max_split = std::min(P.kblocks_total, 64);
        for (int sp = 1; sp <= max_split; ++sp) {
            int per_sp = ceil_div(P.kblocks_total, sp);
            int real = ceil_div(P.kblocks_total, per_sp);  // every slice gets at least one K block
            if (real != sp) continue;
            long long rounds = ceil_div(mn_tiles * sp, P.pair ? sms / 2 : sms);
            double cost = rounds * (per_sp + 4) * block_us;
            if (sp > 1) cost += 3.0 + (2.0 * sp + 1.0) * dw_bytes / 5e6;
            if (best < 0 || cost < best) {
                best = cost;
                split = sp;
            }
        }
    }
    if (P.wpatch) {  // one tile per CTA, no empty slice
        split = std::max(1, std::min(P.kblocks_total, sms / std::max(1, P.n_tiles)));
        split = ceil_div(P.kblocks_total, ceil_div(P.kblocks_total, split));
    }
    P.split_k = split;
    P.num_tiles = mn_tiles * split;
    // One K slice writes dW itself.  Several slices store their partial sums into one fp32 plane each
    // (like dW for the patch walk, else [plain channel][rows of the tile walk]); wgrad_reduce_* then adds
    // the planes in slice order and writes dW once -- no zero-fill, no atomics, bitwise repeatable.
    const size_t dw_elems = static_cast<size_t>(g.plain_c) * g.patch_c * T;
    const int plane_rows = P.wpatch ? 0 : m_tiles * (P.pair ? 2 : 1) * kTileM;
    const size_t plane_elems = (split <= 1) ? 0 : P.wpatch ? round_up(dw_elems, 4) : static_cast<size_t>(g.plain_c) * plane_rows;
    float* planes = (split > 1) ? static_cast<float*>(ws.take(static_cast<size_t>(split) * plane_elems * sizeof(float))) : nullptr;
    if (ws.dry) return NML_OK;
    if (!ws.fits()) return NML_ERR_WORKSPACE;
    P.out = (split > 1) ? planes : g.dw;
    P.plane_elems = plane_elems;
    P.ld_plane = plane_rows;
    // A wave of CTAs re-reads one operand in full; make that the smaller tensor.
    {
        const double patch_bytes = static_cast<double>(g.batch) * g.patch_h * g.patch_w * cpa * mi.es;
        const double plain_bytes = static_cast<double>(g.batch) * g.plain_h * g.plain_w * cpb * mi.es;
        P.m_fastest = (patch_bytes < plain_bytes) ? 1 : 0;
    }

    // MN-major tf32 operands need the 32-byte-chunk swizzle, fp16 ones the plain 128-byte swizzle
    const int mn_swz = (mi.es == 4) ? SWZ_128B_ATOM32 : SWZ_128B;
    for (int pl = 0; pl < mi.planes; ++pl) {
        uint64_t adims[4] = {static_cast<uint64_t>(cpa), static_cast<uint64_t>(g.patch_w),
                             static_cast<uint64_t>(g.patch_h), static_cast<uint64_t>(g.batch)};
        uint32_t abox[4] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>((1 << P.wb_log2) * g.s_w),
                            static_cast<uint32_t>((1 << P.hb_log2) * g.s_h), static_cast<uint32_t>(1 << P.nb_log2)};
        uint32_t aes[4] = {1, static_cast<uint32_t>(g.s_w), static_cast<uint32_t>(g.s_h), 1};
        const int G = kTileM / mi.kb;
        if (P.wpatch) {  // contiguous patch rows; the row stride of the walk lives in the MMA descriptors
            abox[1] = static_cast<uint32_t>(P.patch_w);
            abox[2] = static_cast<uint32_t>(P.patch_h);
            abox[3] = 1;
            aes[1] = aes[2] = 1;
        }
        if (window) {
            uint64_t wd[4] = {64, static_cast<uint64_t>(g.plain_w), static_cast<uint64_t>(wimg.hp), static_cast<uint64_t>(g.batch)};
            uint64_t wstr[3] = {static_cast<uint64_t>(g.s_w) * 16, static_cast<uint64_t>(wimg.wp) * 16,
                                static_cast<uint64_t>(wimg.hp) * wimg.wp * 16};
            uint32_t wbox[4] = {64, static_cast<uint32_t>(1 << P.wb_log2), static_cast<uint32_t>((1 << P.hb_log2) * g.s_h),
                                static_cast<uint32_t>(1 << P.nb_log2)};
            uint32_t wes[4] = {1, 1, static_cast<uint32_t>(g.s_h), 1};
            if (P.wpatch) {
                wbox[1] = abox[1];
                wbox[2] = abox[2];
                wbox[3] = 1;
                wes[2] = 1;
            }
            rc = encode_map(&P.tmA[pl], pa[pl], 2, 4, wd, wbox, wes, mn_swz, wstr);
        } else if (P.wpatch) {
            rc = encode_map(&P.tmA[pl], pa[pl], mi.es, 4, adims, abox, aes, mn_swz);
        } else if (cpa % mi.kb == 0 && P.c_blocks % G == 0) {
            P.a_grouped = 1;
            uint64_t d5[5] = {static_cast<uint64_t>(mi.kb), adims[1], adims[2], adims[3], static_cast<uint64_t>(cpa / mi.kb)};
            uint64_t s5[4] = {static_cast<uint64_t>(cpa) * mi.es, adims[1] * cpa * mi.es, adims[1] * adims[2] * cpa * mi.es,
                              static_cast<uint64_t>(mi.kb) * mi.es};
            uint32_t b5[5] = {abox[0], abox[1], abox[2], abox[3], static_cast<uint32_t>(G)};
            uint32_t e5[5] = {1, aes[1], aes[2], 1, 1};
            rc = encode_map(&P.tmA[pl], pa[pl], mi.es, 5, d5, b5, e5, mn_swz, s5);
        } else {
            rc = encode_map(&P.tmA[pl], pa[pl], mi.es, 4, adims, abox, aes, mn_swz);
        }
        if (rc) return rc;
        uint64_t bdims[4] = {static_cast<uint64_t>(cpb), static_cast<uint64_t>(g.plain_w),
                             static_cast<uint64_t>(g.plain_h), static_cast<uint64_t>(g.batch)};
        uint32_t bbox[4] = {static_cast<uint32_t>(mi.kb), static_cast<uint32_t>(1 << P.wb_log2),
                            static_cast<uint32_t>(1 << P.hb_log2), static_cast<uint32_t>(1 << P.nb_log2)};
        uint32_t bes[4] = {1, 1, 1, 1};
        if (cpb % mi.kb == 0) {
            P.b_grouped = 1;
            uint64_t d5[5] = {static_cast<uint64_t>(mi.kb), bdims[1], bdims[2], bdims[3], static_cast<uint64_t>(cpb / mi.kb)};
            uint64_t s5[4] = {static_cast<uint64_t>(cpb) * mi.es, bdims[1] * cpb * mi.es, bdims[1] * bdims[2] * cpb * mi.es,
                              static_cast<uint64_t>(mi.kb) * mi.es};
            uint32_t b5[5] = {bbox[0], bbox[1], bbox[2], bbox[3], static_cast<uint32_t>((P.pair ? P.bn / 2 : P.bn) / mi.kb)};
            uint32_t e5[5] = {1, 1, 1, 1, 1};
            rc = encode_map(&P.tmB[pl], pb[pl], mi.es, 5, d5, b5, e5, mn_swz, s5);
        } else {
            rc = encode_map(&P.tmB[pl], pb[pl], mi.es, 4, bdims, bbox, bes, mn_swz);
        }
        if (rc) return rc;
    }
    int slot = -1;
    rc = launch_kernel(P, ds, st, &slot);
    if (rc) return rc;
    if (split > 1) {
        const bool vec_ok = (reinterpret_cast<uintptr_t>(g.dw) & 15) == 0;
        if (P.wpatch && vec_ok && dw_elems % 4 == 0 && split > 8) {
            const size_t total4 = dw_elems / 4;
            wgrad_reduce_deep4_kernel<<<static_cast<unsigned>((total4 + 31) / 32), dim3(32, 8), 0, st>>>(planes, g.dw, split, plane_elems, total4);
        } else if (P.wpatch && vec_ok && dw_elems % 4 == 0) {
            const int blocks = static_cast<int>(std::min<size_t>((dw_elems / 4 + 255) / 256, 148 * 8));
            wgrad_reduce_rows4_kernel<<<blocks, 256, 0, st>>>(planes, g.dw, split, plane_elems, 1, static_cast<int>(dw_elems / 4), 0);
        } else if (!P.wpatch && !P.kw_pack && T == 1 && vec_ok && g.patch_c % 4 == 0) {
            const size_t total4 = dw_elems / 4;
            const int blocks = static_cast<int>(std::min<size_t>((total4 + 255) / 256, 148 * 16));
            wgrad_reduce_rows4_kernel<<<blocks, 256, 0, st>>>(planes, g.dw, split, plane_elems, g.plain_c, g.patch_c / 4, plane_rows);
        } else {
            const int layout = P.wpatch ? 0 : P.kw_pack ? 2 : 1;
            const int blocks = static_cast<int>(std::min<size_t>((dw_elems + 255) / 256, 148 * 16));
            wgrad_reduce_kernel<<<blocks, 256, 0, st>>>(planes, g.dw, split, plane_elems, dw_elems, layout, g.patch_c, P.n_taps,
                                                        P.kw_count, P.c_blocks, mi.kb, plane_rows);
        }
        ++g_launches;
        NML_CUDA(cudaGetLastError());
    }
    return profile_stop(slot, st);
}

// --------------------------------------------------------- layer -> problems --
static bool conv_out_size(const nml_conv_desc* d, int* ho, int* wo) {
    if (!d || d->stride_h <= 0 || d->stride_w <= 0 || d->dil_h <= 0 || d->dil_w <= 0 || d->kh <= 0 || d->kw <= 0 ||
        d->pad_h < 0 || d->pad_w < 0)
        return false;
    if (!d->transposed) {
        int nh = d->h + 2 * d->pad_h - d->dil_h * (d->kh - 1) - 1;
        int nw = d->w + 2 * d->pad_w - d->dil_w * (d->kw - 1) - 1;
        if (nh < 0 || nw < 0) return false;
        *ho = nh / d->stride_h + 1;
        *wo = nw / d->stride_w + 1;
    } else {
        *ho = (d->h - 1) * d->stride_h - 2 * d->pad_h + d->dil_h * (d->kh - 1) + 1 + d->outpad_h;
        *wo = (d->w - 1) * d->stride_w - 2 * d->pad_w + d->dil_w * (d->kw - 1) + 1 + d->outpad_w;
    }
    return *ho > 0 && *wo > 0;
}

static int conv_pass(const nml_conv_desc* d, int pass, const void* in0, const void* in1, const void* bias, void* out,
                     float* db, Bump& ws, cudaStream_t st) {
    int ho, wo;
    g_last_scratch_error[0] = 0;  // a workspace error reported from here on is not the static entry point's
    if (!conv_out_size(d, &ho, &wo)) return NML_ERR_INVALID;
    const bool tr = d->transposed != 0;
    if (pass == NML_PASS_BACKWARD_WEIGHT) {
        // in0 = x, in1 = dy
        WgradLike g;
        memset(&g, 0, sizeof(g));
        if (!tr) {
            g.patch = in0; g.patch_c = d->c_in; g.patch_h = d->h; g.patch_w = d->w;
            g.plain = in1; g.plain_c = d->c_out; g.plain_h = ho; g.plain_w = wo;
            g.colsum_of_patch = 0;
        } else {
            g.patch = in1; g.patch_c = d->c_out; g.patch_h = ho; g.patch_w = wo;
            g.plain = in0; g.plain_c = d->c_in; g.plain_h = d->h; g.plain_w = d->w;
            g.colsum_of_patch = 1;
        }
        g.dtype = d->in_dtype; g.layout = d->in_layout; g.batch = d->batch;
        g.kh = d->kh; g.kw = d->kw; g.s_h = d->stride_h; g.s_w = d->stride_w;
        g.p_h = d->pad_h; g.p_w = d->pad_w; g.d_h = d->dil_h; g.d_w = d->dil_w;
        g.dw = static_cast<float*>(out);
        g.colsum = db;
        g.math = d->math;
        return run_wgrad_like(g, ws, st);
    }
    FpropLike f;
    memset(&f, 0, sizeof(f));
    // conv forward and convT backward-data are strided reads; conv backward-data and convT forward gather.
    const bool forward = (pass == NML_PASS_FORWARD);
    const bool reads_layer_input = forward;  // A is the layer input for forward, the output gradient otherwise
    f.a = in0;
    f.a_dtype = d->in_dtype; f.a_layout = d->in_layout; f.batch = d->batch;
    if (reads_layer_input) { f.a_c = d->c_in; f.a_h = d->h; f.a_w = d->w; f.out_c = d->c_out; f.out_h = ho; f.out_w = wo; }
    else                   { f.a_c = d->c_out; f.a_h = ho; f.a_w = wo; f.out_c = d->c_in; f.out_h = d->h; f.out_w = d->w; }
    f.w = in1; f.w_dtype = d->w_dtype;
    // weight source dims: conv [c_out][c_in][T], convT [c_in][c_out][T]
    f.d0 = tr ? d->c_in : d->c_out;
    f.d1 = tr ? d->c_out : d->c_in;
    f.kh = d->kh; f.kw = d->kw;
    // contraction channel is a_c: it is dim0 exactly when a_c names d0
    f.k_is_dim0 = (forward == tr) ? 1 : 0;  // conv fwd: k=c_in=d1; conv bwd: k=c_out=d0; convT fwd: k=c_in=d0; convT bwd: k=c_out=d1
    f.w_direct = 0;
    f.gather = (forward == tr) ? 1 : 0;     // conv fwd 0, conv bwd 1, convT fwd 1, convT bwd 0
    f.s_h = d->stride_h; f.s_w = d->stride_w; f.p_h = d->pad_h; f.p_w = d->pad_w; f.d_h = d->dil_h; f.d_w = d->dil_w;
    f.out = out; f.out_dtype = d->out_dtype; f.out_layout = d->out_layout;
    f.bias = forward ? bias : nullptr; f.bias_dtype = d->w_dtype;
    f.math = d->math;
    f.round_f16 = forward ? d->round_out_f16 : 0;
    return run_fprop_like(f, ws, st);
}

static int linear_pass(const nml_linear_desc* d, int pass, const void* in0, const void* in1, const void* bias,
                       void* out, float* db, Bump& ws, cudaStream_t st) {
    if (!d || d->rows <= 0 || d->in_features <= 0 || d->out_features <= 0) return NML_ERR_INVALID;
    g_last_scratch_error[0] = 0;
    if (pass == NML_PASS_BACKWARD_WEIGHT) {
        WgradLike g;
        memset(&g, 0, sizeof(g));
        g.patch = in0; g.patch_c = d->in_features; g.patch_h = 1; g.patch_w = d->rows;
        g.plain = in1; g.plain_c = d->out_features; g.plain_h = 1; g.plain_w = d->rows;
        g.dtype = d->in_dtype; g.layout = NML_NHWC; g.batch = 1;
        g.kh = g.kw = 1; g.s_h = g.s_w = 1; g.d_h = g.d_w = 1;
        g.dw = static_cast<float*>(out);
        g.colsum = db; g.colsum_of_patch = 0;
        g.math = d->math;
        return run_wgrad_like(g, ws, st);
    }
    FpropLike f;
    memset(&f, 0, sizeof(f));
    const bool forward = (pass == NML_PASS_FORWARD);
    f.a = in0; f.a_dtype = d->in_dtype; f.a_layout = NML_NHWC; f.batch = 1; f.a_h = 1; f.a_w = d->rows;
    f.a_c = forward ? d->in_features : d->out_features;
    f.w = in1; f.w_dtype = d->w_dtype; f.d0 = d->out_features; f.d1 = d->in_features; f.kh = f.kw = 1;
    f.k_is_dim0 = forward ? 0 : 1;
    f.w_direct = 1;
    // Input gradient of a tall layer: W [out][in] read in place is an MN-major B operand, which the tensor core
    // consumes ~10 % slower than a K-major one.  From 8192 rows on, a transposed fp16 copy W^T [in][out] (one
    // coalesced pass over the weights, counted in the pass's duration) pays for itself.
    if (!forward && d->rows >= 8192 && d->math == NML_MATH_F16 && d->w_dtype == NML_F16 && d->in_features % 8 == 0 &&
        d->out_features % 64 == 0 && tune().wtrans) {
        __half* wt = static_cast<__half*>(ws.take(static_cast<size_t>(d->in_features) * d->out_features * sizeof(__half)));
        if (!ws.dry) {
            if (!ws.fits()) return NML_ERR_WORKSPACE;
            int rc = profile_open(st);
            if (rc) return rc;
            const dim3 grid(ceil_div(d->in_features, 64), ceil_div(d->out_features, 64), 1);
            repack_weight_tile_kernel<__half><<<grid, 256, 0, st>>>(static_cast<const __half*>(in1), wt, nullptr, ENC_F16,
                                                                   d->out_features, d->in_features, d->out_features);
            ++g_launches;
            NML_CUDA(cudaGetLastError());
        }
        f.w = wt; f.d0 = d->in_features; f.d1 = d->out_features; f.k_is_dim0 = 0;
    }
    f.gather = 0;
    f.s_h = f.s_w = 1; f.d_h = f.d_w = 1;
    f.out = out; f.out_dtype = d->out_dtype; f.out_layout = NML_NHWC;
    f.out_c = forward ? d->out_features : d->in_features; f.out_h = 1; f.out_w = d->rows;
    f.bias = forward ? bias : nullptr; f.bias_dtype = d->w_dtype;
    f.math = d->math;
    f.round_f16 = forward ? d->round_out_f16 : 0;
    return run_fprop_like(f, ws, st);
}

// Grow-only per-device workspace for the reference-shaped entry points.
struct RefWorkspace {
    void* ptr = nullptr;
    size_t bytes = 0;
};
static RefWorkspace g_ref_ws[64];

static int ref_workspace(size_t need, void** out) {
    int dev = 0;
    NML_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    RefWorkspace& w = g_ref_ws[dev];
    if (need > w.bytes) {
        if (w.ptr) {
            NML_CUDA(cudaDeviceSynchronize());
            NML_CUDA(cudaFree(w.ptr));
            w.ptr = nullptr;
            w.bytes = 0;
        }
        size_t grow = round_up(need + need / 4, 1 << 20);
        NML_CUDA(cudaMalloc(&w.ptr, grow));
        w.bytes = grow;
    }
    *out = w.ptr;
    return NML_OK;
}

// Results of the reference-shaped entry points come from the device's stream-ordered pool
// (cudaMallocAsync on the legacy default stream the entry points run on): no device-wide
// synchronisation per call, freed memory is kept for the next result (release threshold = never).
// cudaFree accepts such pointers, so the reference's own `free_cuda` path keeps working; where a
// device has no memory pools the plain cudaMalloc / cudaFree pair is used.
static bool g_pool_ready[64] = {false};
static bool g_pool_usable[64] = {false};
static int ref_alloc(void** out, size_t bytes) {
    int dev = 0;
    NML_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NML_ERR_INVALID;
    {
        std::lock_guard<std::mutex> lock(g_dev_mutex);
        if (!g_pool_ready[dev]) {
            int supported = 0;
            cudaMemPool_t pool;
            if (cudaDeviceGetAttribute(&supported, cudaDevAttrMemoryPoolsSupported, dev) == cudaSuccess && supported &&
                cudaDeviceGetDefaultMemPool(&pool, dev) == cudaSuccess) {
                unsigned long long keep = ~0ull;
                g_pool_usable[dev] = cudaMemPoolSetAttribute(pool, cudaMemPoolAttrReleaseThreshold, &keep) == cudaSuccess;
            }
            (void)cudaGetLastError();
            g_pool_ready[dev] = true;
        }
    }
    if (g_pool_usable[dev]) NML_CUDA(cudaMallocAsync(out, bytes ? bytes : 1, cudaStreamLegacy));
    else NML_CUDA(cudaMalloc(out, bytes ? bytes : 1));
    return NML_OK;
}
static void ref_release(void* p) {
    int dev = 0;
    if (cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < 64 && g_pool_usable[dev]) cudaFreeAsync(p, cudaStreamLegacy);
    else cudaFree(p);
}

__global__ void tma_box_probe_kernel(const __grid_constant__ CUtensorMap tm, int c0, int c1, int c2, int c3,
                                     uint32_t bytes, uint8_t* out, int* err) {
    extern __shared__ __align__(1024) uint8_t box_smem[];
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(8) int abort_flag[4];
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_state_init(abort_flag, 0);
        fence_mbar_init();
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        mbar_arrive_expect_tx(smem_u32(&bar), bytes);
        tma_load_4d(smem_u32(box_smem), &tm, smem_u32(&bar), c0, c1, c2, c3);
    }
    bool ok = mbar_wait(smem_u32(&bar), 0, abort_flag, err, ERR_WAIT_FULL);
    if (ok)
        for (uint32_t i = threadIdx.x; i < bytes; i += blockDim.x) out[i] = box_smem[i];
}

// One warp waits, with the library's bounded wait, on an mbarrier that nothing ever arrives on.  The
// wait runs out after limit_ns, records ERR_WAIT_FULL in *err and the kernel returns: the give-up path
// of every kernel here, exercised without a fault, a trap or an unbounded spin.
__global__ void wait_limit_probe_kernel(unsigned long long limit_ns, int* err, int* gave_up) {
    __shared__ __align__(8) uint64_t bar;
    __shared__ __align__(8) int abort_flag[4];
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_state_init(abort_flag, limit_ns);
        fence_mbar_init();
    }
    __syncthreads();
    const bool ok = mbar_wait(smem_u32(&bar), 0, abort_flag, err, ERR_WAIT_FULL);
    if (threadIdx.x == 0 && gave_up) *gave_up = ok ? 0 : 1;
}

}  // namespace nml

using namespace nml;

// ---------------------------------------------------------------- C ABI -------
extern "C" {

const char* nml_status_string(int status) {
    switch (status) {
        case NML_OK: return "ok";
        case NML_ERR_INVALID: return "invalid argument";
        case NML_ERR_WORKSPACE: return g_last_scratch_error[0] ? g_last_scratch_error : "workspace too small";
        case NML_ERR_CUDA: return g_last_error[0] ? g_last_error : "CUDA error";
        case NML_ERR_UNSUPPORTED: return "unsupported configuration";
        case NML_ERR_DEVICE: return g_last_device_error[0] ? g_last_device_error : "a kernel abandoned a bounded wait";
    }
    return "unknown status";
}

int nml_conv_output_size(const nml_conv_desc* d, int* h_out, int* w_out) {
    if (!d || !h_out || !w_out) return NML_ERR_INVALID;
    return conv_out_size(d, h_out, w_out) ? NML_OK : NML_ERR_INVALID;
}

int nml_conv_workspace_size(const nml_conv_desc* d, int pass, size_t* bytes) {
    if (!d || !bytes) return NML_ERR_INVALID;
    Bump ws{nullptr, 0, 0, true};
    // (bias and db stand in as non-null so that the scratch behind them is counted)
    float db_stand_in;
    int rc = conv_pass(d, pass, nullptr, nullptr, d, nullptr, &db_stand_in, ws, nullptr);
    *bytes = round_up(ws.off, 256);
    return rc;
}

int nml_linear_workspace_size(const nml_linear_desc* d, int pass, size_t* bytes) {
    if (!d || !bytes) return NML_ERR_INVALID;
    Bump ws{nullptr, 0, 0, true};
    float db_stand_in;
    int rc = linear_pass(d, pass, nullptr, nullptr, d, nullptr, &db_stand_in, ws, nullptr);
    *bytes = round_up(ws.off, 256);
    return rc;
}

int nml_conv_forward(const nml_conv_desc* d, const void* x, const void* w, const void* bias, void* y,
                     void* workspace, size_t workspace_bytes, void* stream) {
    if (!d || !x || !w || !y) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return conv_pass(d, NML_PASS_FORWARD, x, w, bias, y, nullptr, ws, static_cast<cudaStream_t>(stream));
}

int nml_conv_backward_data(const nml_conv_desc* d, const void* dy, const void* w, void* dx, void* workspace,
                           size_t workspace_bytes, void* stream) {
    if (!d || !dy || !w || !dx) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return conv_pass(d, NML_PASS_BACKWARD_DATA, dy, w, nullptr, dx, nullptr, ws, static_cast<cudaStream_t>(stream));
}

int nml_conv_backward_weight(const nml_conv_desc* d, const void* x, const void* dy, float* dw, float* db,
                             void* workspace, size_t workspace_bytes, void* stream) {
    if (!d || !x || !dy || !dw) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return conv_pass(d, NML_PASS_BACKWARD_WEIGHT, x, dy, nullptr, dw, db, ws, static_cast<cudaStream_t>(stream));
}

int nml_linear_forward(const nml_linear_desc* d, const void* x, const void* w, const void* bias, void* y,
                       void* workspace, size_t workspace_bytes, void* stream) {
    if (!d || !x || !w || !y) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return linear_pass(d, NML_PASS_FORWARD, x, w, bias, y, nullptr, ws, static_cast<cudaStream_t>(stream));
}

int nml_linear_backward_data(const nml_linear_desc* d, const void* dy, const void* w, void* dx, void* workspace,
                             size_t workspace_bytes, void* stream) {
    if (!d || !dy || !w || !dx) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return linear_pass(d, NML_PASS_BACKWARD_DATA, dy, w, nullptr, dx, nullptr, ws,
                       static_cast<cudaStream_t>(stream));
}

int nml_linear_backward_weight(const nml_linear_desc* d, const void* x, const void* dy, float* dw, float* db,
                               void* workspace, size_t workspace_bytes, void* stream) {
    if (!d || !x || !dy || !dw) return NML_ERR_INVALID;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    return linear_pass(d, NML_PASS_BACKWARD_WEIGHT, x, dy, nullptr, dw, db, ws, static_cast<cudaStream_t>(stream));
}

int nml_set_sm_limit(int sms) {
    if (sms < 0) return NML_ERR_INVALID;
    g_sm_limit.store(sms);
    return NML_OK;
}

int nml_init(void) {
    DeviceState* ds = nullptr;
    return device_state(&ds);
}

// Reads and clears one status word; the code of an abandoned wait goes into *code and into the
// message nml_status_string returns for NML_ERR_DEVICE.
static int read_status_word(int* word, int* code) {
    NML_CUDA(cudaDeviceSynchronize());
    int v = 0;
    NML_CUDA(cudaMemcpy(&v, word, sizeof(int), cudaMemcpyDeviceToHost));
    if (code) *code = v;
    if (v == 0) return NML_OK;
    NML_CUDA(cudaMemset(word, 0, sizeof(int)));
    snprintf(g_last_device_error, sizeof(g_last_device_error), "a kernel abandoned bounded wait %d (%s)", v,
             v == ERR_WAIT_EMPTY ? "producer: free stage" : v == ERR_WAIT_FULL ? "operands to land"
             : v == ERR_WAIT_TMEM_EMPTY ? "accumulator to drain" : v == ERR_WAIT_TMEM_FULL ? "accumulator to fill"
             : v == ERR_WAIT_DRAIN ? "copies in flight at unwinding" : "unknown");
    return NML_ERR_DEVICE;
}

int nml_device_status(int* code) {
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    return read_status_word(ds->err, code);
}

long long nml_launch_count(void) { return g_launches.load() + nml_layers_launch_count(); }

int nml_profile_begin(int max_records) {
    if (max_records <= 0 || max_records > 1 << 16) return NML_ERR_INVALID;
    while (static_cast<int>(g_prof.start.size()) < max_records) {
        cudaEvent_t a, b;
        NML_CUDA(cudaEventCreate(&a));
        NML_CUDA(cudaEventCreate(&b));
        g_prof.start.push_back(a);
        g_prof.stop.push_back(b);
    }
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    g_prof.cap = max_records;
    g_prof.n = 0;
    g_prof.on = true;
    return NML_OK;
}

int nml_profile_end(float* ms_out, int capacity, int* count) {
    if (!ms_out || !count) return NML_ERR_INVALID;
    g_prof.on = false;
    NML_CUDA(cudaDeviceSynchronize());
    int n = std::min(g_prof.n, capacity);
    for (int i = 0; i < n; ++i) NML_CUDA(cudaEventElapsedTime(&ms_out[i], g_prof.start[i], g_prof.stop[i]));
    *count = n;
    return NML_OK;
}

// ---- forward entry point that allocates nothing ----
// Scratch for the converted operands lives in the library image instead of caller memory.
// kStaticScratchBytes of every GPU that loads this library are held until the process exits.
constexpr size_t kStaticScratchBytes = 64ull << 20;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];
static __device__ int g_static_status;  // where kernels launched by this entry point report a give-up (see g_status_word)

struct StaticState {
    bool ready = false;
    void* scratch = nullptr;  // DEVICE address of g_static_scratch on this device
    DeviceState ds;           // status word = device address of g_static_status
};
static StaticState g_static[64];

// Once per device, with that device current.  In host code `g_static_scratch` is only a handle for
// the symbol, not an address a kernel may use: the device address comes from cudaGetSymbolAddress.
static int static_state(StaticState** out) {
    int dev = 0;
    NML_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return NML_ERR_INVALID;
    std::lock_guard<std::mutex> lock(g_dev_mutex);
    StaticState& s = g_static[dev];
    if (!s.ready) {
        void* scratch = nullptr;
        void* status = nullptr;
        NML_CUDA(cudaGetSymbolAddress(&scratch, g_static_scratch));
        NML_CUDA(cudaGetSymbolAddress(&status, g_static_status));
        NML_CUDA(cudaMemset(status, 0, sizeof(int)));
        NML_CUDA(cudaDeviceGetAttribute(&s.ds.sms, cudaDevAttrMultiProcessorCount, dev));
        int rc_attr = raise_smem_limit();
        if (rc_attr) return rc_attr;
        rc_attr = load_helper_kernels();  // so that no later call is the first use (= the loading) of a kernel
        if (rc_attr) return rc_attr;
        s.scratch = scratch;
        s.ds.err = static_cast<int*>(status);
        s.ds.attr_set = true;
        s.ready = true;
    }
    *out = &s;
    return NML_OK;
}

int nml_conv_forward_static(const nml_conv_desc* d, const void* x, const void* w, const void* bias, void* y,
                            void* stream) {
    StaticState* ss = nullptr;
    if (!d) {  // query form: wait for the device, report and clear a recorded give-up
        int rc = static_state(&ss);
        if (rc) return rc;
        return read_status_word(ss->ds.err, nullptr);  // the code is in nml_status_string(NML_ERR_DEVICE)
    }
    if (!x || !w || !y) return NML_ERR_INVALID;
    Bump dry{nullptr, 0, 0, true};
    int rc = conv_pass(d, NML_PASS_FORWARD, nullptr, nullptr, bias ? d : nullptr, nullptr, nullptr, dry, nullptr);
    if (rc) return rc;
    const size_t need = round_up(dry.off, 256);
    if (need > kStaticScratchBytes) {
        snprintf(g_last_scratch_error, sizeof(g_last_scratch_error),
                 "this layer needs %zu bytes of scratch; the built-in scratch array holds %zu "
                 "(use nml_conv_forward with a caller workspace)", need, kStaticScratchBytes);
        return NML_ERR_WORKSPACE;
    }
    rc = static_state(&ss);
    if (rc) return rc;
    // Every region of the scratch that the contraction reads is rewritten in full by the conversion
    // passes of this call (channel and K padding included), so nothing from the last call survives.
    Bump ws{static_cast<uint8_t*>(ss->scratch), 0, kStaticScratchBytes, false, &ss->ds};
    return conv_pass(d, NML_PASS_FORWARD, x, w, bias, y, nullptr, ws, static_cast<cudaStream_t>(stream));
}

// ---- reference-shaped entry points ----
static void fill_conv_desc(nml_conv_desc* d, int transposed, int B, int C_in, int H, int W, int C_out, int KH,
                           int KW, int sh, int sw, int ph, int pw, int dh, int dw, int oph, int opw) {
    memset(d, 0, sizeof(*d));
    d->batch = B; d->c_in = C_in; d->h = H; d->w = W; d->c_out = C_out; d->kh = KH; d->kw = KW;
    d->stride_h = sh; d->stride_w = sw; d->pad_h = ph; d->pad_w = pw; d->dil_h = dh; d->dil_w = dw;
    d->outpad_h = oph; d->outpad_w = opw; d->transposed = transposed;
    d->in_layout = d->out_layout = NML_NCHW;
}

static int ref_run_conv(nml_conv_desc* d, int pass, const void* in0, const void* in1, const void* bias,
                        size_t out_bytes, uintptr_t* result) {
    if (!result) return NML_ERR_INVALID;
    size_t need = 0;
    int rc = nml_conv_workspace_size(d, pass, &need);
    if (rc) return rc;
    void* ws = nullptr;
    rc = ref_workspace(need, &ws);
    if (rc) return rc;
    void* out = nullptr;
    rc = ref_alloc(&out, out_bytes);
    if (rc) return rc;
    Bump b{static_cast<uint8_t*>(ws), 0, need, false};
    rc = conv_pass(d, pass, in0, in1, bias, out, nullptr, b, nullptr);
    if (rc) {
        ref_release(out);
        return rc;
    }
    *result = reinterpret_cast<uintptr_t>(out);
    return NML_OK;
}

static int ref_forward(int transposed, uintptr_t input_ptr, uintptr_t weight_ptr, uintptr_t bias_ptr,
                       size_t output_size, int B, int C_in, int H, int W, int C_out, int KH, int KW, int sh, int sw,
                       int ph, int pw, int dh, int dw, int oph, int opw, int groups, int dtype, int half_precision,
                       uintptr_t* result) {
    if (groups != 1) return NML_ERR_UNSUPPORTED;
    if (dtype != NML_F32 && dtype != NML_F16) return NML_ERR_INVALID;
    nml_conv_desc d;
    fill_conv_desc(&d, transposed, B, C_in, H, W, C_out, KH, KW, sh, sw, ph, pw, dh, dw, oph, opw);
    d.in_dtype = d.out_dtype = d.w_dtype = dtype;
    d.math = (half_precision || dtype == NML_F16) ? NML_MATH_F16 : NML_MATH_3XTF32;
    d.round_out_f16 = half_precision ? 1 : 0;
    int ho, wo;
    if (!conv_out_size(&d, &ho, &wo)) return NML_ERR_INVALID;
    size_t elems = static_cast<size_t>(B) * C_out * ho * wo;
    if (output_size != 0 && output_size != elems) return NML_ERR_INVALID;
    return ref_run_conv(&d, NML_PASS_FORWARD, reinterpret_cast<const void*>(input_ptr),
                        reinterpret_cast<const void*>(weight_ptr), reinterpret_cast<const void*>(bias_ptr),
                        elems * (dtype == NML_F16 ? 2 : 4), result);
}

int nml_ref_conv2d(uintptr_t input_ptr, size_t input_size, uintptr_t weight_ptr, size_t weight_size,
                   uintptr_t bias_ptr, size_t bias_size, size_t output_size, int B, int C_in, int H, int W, int C_out,
                   int KH, int KW, int stride_h, int stride_w, int padding_h, int padding_w, int dilation_h,
                   int dilation_w, int groups, int dtype, int half_precision, uintptr_t* result) {
    (void)input_size; (void)weight_size; (void)bias_size;
    return ref_forward(0, input_ptr, weight_ptr, bias_ptr, output_size, B, C_in, H, W, C_out, KH, KW, stride_h,
                       stride_w, padding_h, padding_w, dilation_h, dilation_w, 0, 0, groups, dtype, half_precision,
                       result);
}

int nml_ref_conv_transpose2d(uintptr_t input_ptr, size_t input_size, uintptr_t weight_ptr, size_t weight_size,
                             uintptr_t bias_ptr, size_t bias_size, size_t output_size, int B, int C_in, int H, int W,
                             int C_out, int KH, int KW, int stride_h, int stride_w, int padding_h, int padding_w,
                             int dilation_h, int dilation_w, int output_padding_h, int output_padding_w, int groups,
                             int dtype, int half_precision, uintptr_t* result) {
    (void)input_size; (void)weight_size; (void)bias_size;
    return ref_forward(1, input_ptr, weight_ptr, bias_ptr, output_size, B, C_in, H, W, C_out, KH, KW, stride_h,
                       stride_w, padding_h, padding_w, dilation_h, dilation_w, output_padding_h, output_padding_w,
                       groups, dtype, half_precision, result);
}

// The backward entry points receive H_out/W_out explicitly; for ConvTranspose2d they determine
// the output padding, which the reference's signature does not pass.
static int ref_backward(int transposed, int pass, uintptr_t p0, uintptr_t p1, int B, int C_in, int H, int W,
                        int C_out, int KH, int KW, int H_out, int W_out, int sh, int sw, int ph, int pw, int dh,
                        int dw, int dtype, uintptr_t* result) {
    if (dtype != NML_F32 && dtype != NML_F16) return NML_ERR_INVALID;
    nml_conv_desc d;
    fill_conv_desc(&d, transposed, B, C_in, H, W, C_out, KH, KW, sh, sw, ph, pw, dh, dw, 0, 0);
    int ho, wo;
    if (!conv_out_size(&d, &ho, &wo)) return NML_ERR_INVALID;
    if (transposed) {
        d.outpad_h = H_out - ho;
        d.outpad_w = W_out - wo;
        if (d.outpad_h < 0 || d.outpad_w < 0 || d.outpad_h >= sh + dh || d.outpad_w >= sw + dw) return NML_ERR_INVALID;
    } else if (ho != H_out || wo != W_out) {
        return NML_ERR_INVALID;
    }
    d.in_dtype = d.w_dtype = dtype;
    d.out_dtype = NML_F32;
    d.math = (dtype == NML_F16) ? NML_MATH_F16 : NML_MATH_3XTF32;
    size_t elems;
    const void *in0, *in1;
    if (pass == NML_PASS_BACKWARD_DATA) {
        elems = static_cast<size_t>(B) * C_in * H * W;
        in0 = reinterpret_cast<const void*>(p0);  // out_grad
        in1 = reinterpret_cast<const void*>(p1);  // weight
    } else {
        elems = static_cast<size_t>(C_out) * C_in * KH * KW;
        in0 = reinterpret_cast<const void*>(p1);  // input
        in1 = reinterpret_cast<const void*>(p0);  // out_grad
    }
    return ref_run_conv(&d, pass, in0, in1, nullptr, elems * 4, result);
}

int nml_ref_conv2d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int H, int W,
                                  int C_out, int KH, int KW, int H_out, int W_out, int stride_h, int stride_w,
                                  int padding_h, int padding_w, int dilation_h, int dilation_w, int groups, int dtype,
                                  uintptr_t* result) {
    if (groups != 1) return NML_ERR_UNSUPPORTED;
    return ref_backward(0, NML_PASS_BACKWARD_DATA, out_grad_ptr, weight_ptr, B, C_in, H, W, C_out, KH, KW, H_out,
                        W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, dtype, result);
}

int nml_ref_conv_transpose2d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int H,
                                            int W, int C_out, int KH, int KW, int H_out, int W_out, int stride_h,
                                            int stride_w, int padding_h, int padding_w, int dilation_h,
                                            int dilation_w, int groups, int dtype, uintptr_t* result) {
    if (groups != 1) return NML_ERR_UNSUPPORTED;
    return ref_backward(1, NML_PASS_BACKWARD_DATA, out_grad_ptr, weight_ptr, B, C_in, H, W, C_out, KH, KW, H_out,
                        W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, dtype, result);
}

int nml_ref_conv2d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int H, int W,
                                   int C_out, int KH, int KW, int H_out, int W_out, int stride_h, int stride_w,
                                   int padding_h, int padding_w, int dilation_h, int dilation_w, int dtype,
                                   uintptr_t* result) {
    return ref_backward(0, NML_PASS_BACKWARD_WEIGHT, out_grad_ptr, input_ptr, B, C_in, H, W, C_out, KH, KW, H_out,
                        W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, dtype, result);
}

int nml_ref_conv_transpose2d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int H,
                                             int W, int C_out, int KH, int KW, int H_out, int W_out, int stride_h,
                                             int stride_w, int padding_h, int padding_w, int dilation_h,
                                             int dilation_w, int dtype, uintptr_t* result) {
    return ref_backward(1, NML_PASS_BACKWARD_WEIGHT, out_grad_ptr, input_ptr, B, C_in, H, W, C_out, KH, KW, H_out,
                        W_out, stride_h, stride_w, padding_h, padding_w, dilation_h, dilation_w, dtype, result);
}

// 1-D convolutions are the same walks over an image of height 1 ([B, C, L] is [B, C, 1, L]).
int nml_ref_conv1d(uintptr_t input_ptr, uintptr_t weight_ptr, uintptr_t bias_ptr, int B, int C_in, int L, int C_out,
                   int K, int stride, int padding, int dilation, int groups, int dtype, uintptr_t* result) {
    return ref_forward(0, input_ptr, weight_ptr, bias_ptr, 0, B, C_in, 1, L, C_out, 1, K, 1, stride, 0, padding, 1,
                       dilation, 0, 0, groups, dtype, 0, result);
}

int nml_ref_conv_transpose1d(uintptr_t input_ptr, uintptr_t weight_ptr, uintptr_t bias_ptr, int B, int C_in, int L,
                             int C_out, int K, int stride, int padding, int dilation, int output_padding, int groups,
                             int dtype, uintptr_t* result) {
    return ref_forward(1, input_ptr, weight_ptr, bias_ptr, 0, B, C_in, 1, L, C_out, 1, K, 1, stride, 0, padding, 1,
                       dilation, 0, output_padding, groups, dtype, 0, result);
}

int nml_ref_conv1d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int L, int C_out,
                                  int K, int L_out, int stride, int padding, int dilation, int groups, int dtype,
                                  uintptr_t* result) {
    if (groups != 1) return NML_ERR_UNSUPPORTED;
    return ref_backward(0, NML_PASS_BACKWARD_DATA, out_grad_ptr, weight_ptr, B, C_in, 1, L, C_out, 1, K, 1, L_out, 1,
                        stride, 0, padding, 1, dilation, dtype, result);
}

int nml_ref_conv_transpose1d_backward_input(uintptr_t out_grad_ptr, uintptr_t weight_ptr, int B, int C_in, int L,
                                            int C_out, int K, int L_out, int stride, int padding, int dilation,
                                            int groups, int dtype, uintptr_t* result) {
    if (groups != 1) return NML_ERR_UNSUPPORTED;
    return ref_backward(1, NML_PASS_BACKWARD_DATA, out_grad_ptr, weight_ptr, B, C_in, 1, L, C_out, 1, K, 1, L_out, 1,
                        stride, 0, padding, 1, dilation, dtype, result);
}

int nml_ref_conv1d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int L, int C_out,
                                   int K, int L_out, int stride, int padding, int dilation, int dtype,
                                   uintptr_t* result) {
    return ref_backward(0, NML_PASS_BACKWARD_WEIGHT, out_grad_ptr, input_ptr, B, C_in, 1, L, C_out, 1, K, 1, L_out, 1,
                        stride, 0, padding, 1, dilation, dtype, result);
}

int nml_ref_conv_transpose1d_backward_weight(uintptr_t out_grad_ptr, uintptr_t input_ptr, int B, int C_in, int L,
                                             int C_out, int K, int L_out, int stride, int padding, int dilation,
                                             int dtype, uintptr_t* result) {
    return ref_backward(1, NML_PASS_BACKWARD_WEIGHT, out_grad_ptr, input_ptr, B, C_in, 1, L, C_out, 1, K, 1, L_out, 1,
                        stride, 0, padding, 1, dilation, dtype, result);
}

int nml_ref_matmul(uintptr_t a_ptr, uintptr_t b_ptr, const int* a_shape, int a_rank, const int* b_shape, int b_rank,
                   int dtype, uintptr_t* result) {
    if (!a_shape || !b_shape || a_rank < 2 || b_rank < 2 || !result) return NML_ERR_INVALID;
    if (dtype != NML_F32 && dtype != NML_F16) return NML_ERR_INVALID;
    const int M = a_shape[a_rank - 2], K = a_shape[a_rank - 1], N = b_shape[b_rank - 1];
    if (b_shape[b_rank - 2] != K) return NML_ERR_INVALID;
    size_t batch = 1;
    for (int i = 0; i < a_rank - 2; ++i) batch *= a_shape[i];
    size_t b_batch = 1;
    for (int i = 0; i < b_rank - 2; ++i) b_batch *= b_shape[i];
    // A 2-D right operand is shared by every batch entry; a batched one must match.
    if (b_batch != 1 && b_batch != batch) return NML_ERR_INVALID;
    const int es = (dtype == NML_F16) ? 2 : 4;
    // C = A * B with B [K][N]: the backward-data form of a Linear layer whose weight is B.
    nml_linear_desc d;
    memset(&d, 0, sizeof(d));
    d.rows = M; d.out_features = K; d.in_features = N;
    d.in_dtype = d.out_dtype = d.w_dtype = dtype;
    d.math = (dtype == NML_F16) ? NML_MATH_F16 : NML_MATH_3XTF32;
    size_t need = 0;
    int rc = nml_linear_workspace_size(&d, NML_PASS_BACKWARD_DATA, &need);
    if (rc) return rc;
    void* ws = nullptr;
    rc = ref_workspace(need, &ws);
    if (rc) return rc;
    void* out = nullptr;
    rc = ref_alloc(&out, batch * M * N * es);
    if (rc) return rc;
    for (size_t b = 0; b < batch; ++b) {
        const uint8_t* A = reinterpret_cast<const uint8_t*>(a_ptr) + b * M * K * es;
        const uint8_t* Bm = reinterpret_cast<const uint8_t*>(b_ptr) + (b_batch == 1 ? 0 : b) * K * N * es;
        uint8_t* C = static_cast<uint8_t*>(out) + b * M * N * es;
        Bump bump{static_cast<uint8_t*>(ws), 0, need, false};
        rc = linear_pass(&d, NML_PASS_BACKWARD_DATA, A, Bm, nullptr, C, nullptr, bump, nullptr);
        if (rc) {
            ref_release(out);
            return rc;
        }
    }
    *result = reinterpret_cast<uintptr_t>(out);
    return NML_OK;
}

int nml_ref_free(uintptr_t ptr) {
    if (ptr) ref_release(reinterpret_cast<void*>(ptr));
    NML_CUDA(cudaGetLastError());
    return NML_OK;
}

int nml_debug_tma_box(const void* tensor, int elem_bytes, const int dims[4], const int box[4],
                      const int elem_strides[4], const int coords[4], void* out, size_t out_bytes, void* stream) {
    if (!tensor || !out || (elem_bytes != 2 && elem_bytes != 4)) return NML_ERR_INVALID;
    DeviceState* ds = nullptr;
    int rc = device_state(&ds);
    if (rc) return rc;
    uint64_t gd[4];
    uint32_t bx[4], es[4];
    size_t bytes = elem_bytes;
    for (int i = 0; i < 4; ++i) {
        gd[i] = dims[i];
        bx[i] = box[i];
        es[i] = elem_strides[i];
        bytes *= (box[i] + elem_strides[i] - 1) / elem_strides[i];
    }
    if (bytes > 96 * 1024 || bytes > out_bytes || bytes % 16) return NML_ERR_INVALID;
    CUtensorMap tm;
    rc = encode_map(&tm, tensor, elem_bytes, 4, gd, bx, es, SWZ_NONE);
    if (rc) return rc;
    static bool attr = false;
    if (!attr) {
        NML_CUDA(cudaFuncSetAttribute(tma_box_probe_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024));
        attr = true;
    }
    tma_box_probe_kernel<<<1, 128, bytes + 1024, static_cast<cudaStream_t>(stream)>>>(
        tm, coords[0], coords[1], coords[2], coords[3], static_cast<uint32_t>(bytes), static_cast<uint8_t*>(out),
        ds->err);
    NML_CUDA(cudaGetLastError());
    return NML_OK;
}

int nml_debug_wait_timeout(unsigned long long limit_ns, int use_static_word, void* stream) {
    if (limit_ns == 0 || limit_ns > 100000000ull) return NML_ERR_INVALID;  // at most 0.1 s
    int* word = nullptr;
    if (use_static_word) {
        StaticState* ss = nullptr;
        int rc = static_state(&ss);
        if (rc) return rc;
        word = ss->ds.err;
    } else {
        DeviceState* ds = nullptr;
        int rc = device_state(&ds);
        if (rc) return rc;
        word = ds->err;
    }
    wait_limit_probe_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns, word, nullptr);
    NML_CUDA(cudaGetLastError());
    return NML_OK;
}

int nml_debug_stalled_linear_forward(const nml_linear_desc* d, const void* x, const void* w, void* y, void* workspace,
                                     size_t workspace_bytes, unsigned long long limit_ns, void* stream) {
    if (!d || !x || !w || !y || limit_ns == 0 || limit_ns > 100000000ull) return NML_ERR_INVALID;
    // only the plain stage-ring walk of a small fp16 layer (one CTA per tile, no pairs): every wait in it is
    // bounded and no MMA is ever issued
    if (d->math != NML_MATH_F16 || d->in_dtype != NML_F16 || d->w_dtype != NML_F16 || d->rows > 4096 ||
        d->in_features > 1024 || d->out_features > 128 || d->in_features % 8 || d->out_features % 8)
        return NML_ERR_UNSUPPORTED;
    Bump ws{static_cast<uint8_t*>(workspace), 0, workspace ? workspace_bytes : 0, false};
    g_dbg_wait_limit_ns = limit_ns;
    g_dbg_short_a_box = true;
    int rc = linear_pass(d, NML_PASS_FORWARD, x, w, nullptr, y, nullptr, ws, static_cast<cudaStream_t>(stream));
    g_dbg_wait_limit_ns = 0;
    g_dbg_short_a_box = false;
    return rc;
}

int nml_debug_copy_to_host(void* host_dst, uintptr_t device_src, size_t bytes) {
    if (!host_dst || !device_src) return NML_ERR_INVALID;
    NML_CUDA(cudaMemcpy(host_dst, reinterpret_cast<const void*>(device_src), bytes, cudaMemcpyDeviceToHost));
    return NML_OK;
}

}  // extern "C"
