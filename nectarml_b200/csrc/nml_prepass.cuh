// Memory-bound helper kernels around the contraction kernel: layout / precision
// conversion of activations (NCHW -> NHWC, fp32 -> fp16 or the tf32 hi/lo pair of the
// 3xTF32 split, with the bias-gradient column sum folded into the same pass over dY),
// weight repacking into the K-major [n][tap][k] operand, and small utilities.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace nml {

__device__ __forceinline__ float to_tf32_rna(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return __uint_as_float(r);
}

__device__ __forceinline__ float load_as_float(const float* p, size_t i) { return p[i]; }
__device__ __forceinline__ float load_as_float(const __half* p, size_t i) { return __half2float(p[i]); }

// Output encodings of the conversion kernels.
enum { ENC_F16 = 0, ENC_TF32_PAIR = 1, ENC_TF32_HI = 2 };

__device__ __forceinline__ void store_enc(int enc, void* out0, void* out1, size_t i, float v) {
    if (enc == ENC_F16) {
        reinterpret_cast<__half*>(out0)[i] = __float2half_rn(v);
    } else {
        float hi = to_tf32_rna(v);
        reinterpret_cast<float*>(out0)[i] = hi;
        if (enc == ENC_TF32_PAIR) reinterpret_cast<float*>(out1)[i] = to_tf32_rna(v - hi);
    }
}

// in  [N][C][HW] (NCHW)  ->  out [N][HW][Cp] (NHWC, channels zero-padded to Cp).
// Tile of 64 channels x 64 pixels through shared memory.  Loads run along pixels (one 256-byte
// row segment per 16 threads when the rows allow 16-byte loads), stores along channels: 8 threads
// write the 64 channels of one pixel as 16-byte (fp16) or 2 x 16-byte (tf32 planes) pieces, so a
// warp store covers four whole pixels.  When `colsum` is given, the per-channel sums over the tile's
// pixels (a share of the bias gradient) go to row (n * gridDim.x + blockIdx.x) of that [tiles][C]
// matrix of partial sums; colsum_finish_kernel adds the rows in a fixed order (no atomics, so the
// bias gradient is bitwise repeatable).
template <typename TIn>
__global__ void __launch_bounds__(256) nchw_to_nhwc_kernel(const TIn* __restrict__ in, void* out0,
                                                           void* out1, int enc, int C, int Cp, int HW,
                                                           float* colsum) {
    __shared__ float tile[64][65];
    const int n = blockIdx.z;
    const int c0 = blockIdx.y * 64;
    const int p0 = blockIdx.x * 64;
    const TIn* src = in + static_cast<size_t>(n) * C * HW;
    const bool vec_ok = (sizeof(TIn) == 4) && (HW % 4 == 0) && ((reinterpret_cast<uintptr_t>(in) & 15) == 0);
    if (vec_ok) {
        const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;  // 16 x 16: four pixels per thread
        for (int c = ty; c < 64; c += 16) {
            float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
            const int p = p0 + 4 * tx;
            if (c0 + c < C && p < HW)  // HW % 4 == 0, so a started quad is complete
                v = __ldg(reinterpret_cast<const float4*>(reinterpret_cast<const float*>(src) +
                                                          static_cast<size_t>(c0 + c) * HW + p));
            tile[c][4 * tx + 0] = v.x;
            tile[c][4 * tx + 1] = v.y;
            tile[c][4 * tx + 2] = v.z;
            tile[c][4 * tx + 3] = v.w;
        }
    } else {
        const int tx = threadIdx.x & 63, ty = threadIdx.x >> 6;  // 64 x 4
        for (int c = ty; c < 64; c += 4) {
            float v = 0.f;
            if (c0 + c < C && p0 + tx < HW) v = load_as_float(src, static_cast<size_t>(c0 + c) * HW + p0 + tx);
            tile[c][tx] = v;
        }
    }
    __syncthreads();
    if (colsum != nullptr && threadIdx.x < 64 && c0 + threadIdx.x < C) {
        float s = 0.f;
        for (int p = 0; p < 64; ++p) s += tile[threadIdx.x][(p + threadIdx.x) & 63];
        colsum[(static_cast<size_t>(n) * gridDim.x + blockIdx.x) * C + c0 + threadIdx.x] = s;
    }
    // store: 8 threads per pixel, 8 channels each
    const int j = threadIdx.x & 7, pp = threadIdx.x >> 3;  // 8 x 32
    const int cb = c0 + 8 * j;
    const bool full8 = (cb + 8 <= Cp) && (Cp % 8 == 0);
    for (int p = pp; p < 64; p += 32) {
        if (p0 + p >= HW || cb >= Cp) continue;
        const size_t o = (static_cast<size_t>(n) * HW + p0 + p) * Cp + cb;
        float v[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) v[i] = tile[8 * j + i][p];
        if (full8 && enc == ENC_F16) {
            uint4 pk;
            __half2 h;
            h = __floats2half2_rn(v[0], v[1]); pk.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[2], v[3]); pk.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[4], v[5]); pk.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(v[6], v[7]); pk.w = *reinterpret_cast<uint32_t*>(&h);
            *reinterpret_cast<uint4*>(reinterpret_cast<__half*>(out0) + o) = pk;
        } else if (full8) {
            float hi[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) hi[i] = to_tf32_rna(v[i]);
            float4* d0 = reinterpret_cast<float4*>(reinterpret_cast<float*>(out0) + o);
            d0[0] = make_float4(hi[0], hi[1], hi[2], hi[3]);
            d0[1] = make_float4(hi[4], hi[5], hi[6], hi[7]);
            if (enc == ENC_TF32_PAIR) {
                float4* d1 = reinterpret_cast<float4*>(reinterpret_cast<float*>(out1) + o);
                d1[0] = make_float4(to_tf32_rna(v[0] - hi[0]), to_tf32_rna(v[1] - hi[1]), to_tf32_rna(v[2] - hi[2]),
                                    to_tf32_rna(v[3] - hi[3]));
                d1[1] = make_float4(to_tf32_rna(v[4] - hi[4]), to_tf32_rna(v[5] - hi[5]), to_tf32_rna(v[6] - hi[6]),
                                    to_tf32_rna(v[7] - hi[7]));
            }
        } else {
            for (int i = 0; i < 8 && cb + i < Cp; ++i) store_enc(enc, out0, out1, o + i, v[i]);
        }
    }
}

// Row-major [R][C] -> [R][Cp] with encoding change (fp32/fp16 -> fp16 / tf32 pair), zero pad.
template <typename TIn>
__global__ void __launch_bounds__(256) convert_rows_kernel(const TIn* __restrict__ in, void* out0,
                                                           void* out1, int enc, size_t R, int C, int Cp) {
    size_t total = R * static_cast<size_t>(Cp);
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t r = i / Cp;
        int c = static_cast<int>(i - r * Cp);
        float v = (c < C) ? load_as_float(in, r * C + c) : 0.f;
        store_enc(enc, out0, out1, i, v);
    }
}

// Column sums of a row-major [R][C] matrix (bias gradient of Linear, or of an NHWC dY), first stage:
// row block blockIdx.y writes its sums to row blockIdx.y of the [row blocks][C] partial-sum matrix.
template <typename TIn>
__global__ void __launch_bounds__(256) colsum_rows_kernel(const TIn* __restrict__ in, float* colsum,
                                                          size_t R, int C, int rows_per_block) {
    size_t r0 = static_cast<size_t>(blockIdx.y) * rows_per_block;
    size_t r1 = r0 + rows_per_block < R ? r0 + rows_per_block : R;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < C; c += gridDim.x * blockDim.x) {
        float s = 0.f;
        for (size_t r = r0; r < r1; ++r) s += load_as_float(in, r * C + c);
        colsum[static_cast<size_t>(blockIdx.y) * C + c] = s;
    }
}

// Vectorised column sums for fp16 rows whose length is a multiple of 8: every thread owns 8
// adjacent columns (one 16-byte load per row), a warp covers 256 columns, blockDim.y warps take
// interleaved rows, and each block writes its partial sums to its row of the partial-sum matrix.
__global__ void __launch_bounds__(256) colsum_rows_f16x8_kernel(const __half* __restrict__ in, float* colsum,
                                                                size_t R, int C, int rows_per_block) {
    __shared__ float part[8][256];
    const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
    const int c0 = (blockIdx.x * 32 + lane) * 8;
    size_t r0 = static_cast<size_t>(blockIdx.y) * rows_per_block;
    size_t r1 = r0 + rows_per_block < R ? r0 + rows_per_block : R;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (c0 < C) {
#pragma unroll 4  // several 16-byte loads in flight per thread: the pass is HBM-bound
        for (size_t r = r0 + wy; r < r1; r += 8) {
            uint4 v = __ldg(reinterpret_cast<const uint4*>(in + r * C + c0));
            const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                float2 f = __half22float2(h[j]);
                acc[2 * j] += f.x;
                acc[2 * j + 1] += f.y;
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) part[wy][lane * 8 + j] = acc[j];
    __syncthreads();
    const int c = blockIdx.x * 256 + threadIdx.x;
    if (c < C) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) sum += part[w][threadIdx.x];
        colsum[static_cast<size_t>(blockIdx.y) * C + c] = sum;
    }
}

// Weights [D0][D1][T] -> K-major operand dst[n][t][kp]:
//   k_is_dim0 == 0 : n = D0 index, k = D1 index   (Conv2d forward, ConvTranspose2d dgrad)
//   k_is_dim0 == 1 : n = D1 index, k = D0 index   (Conv2d dgrad, ConvTranspose2d forward)
// k is zero-padded to kp per tap so that no K block straddles two taps.  Both cases swap the two inner
// dimensions of a [B][R][Cc] array: out[b][c][r] = in[b][r][c], rows padded to Rp --
//   k_is_dim0 == 0 : B = D0, R = D1 (k), Cc = T          k_is_dim0 == 1 : B = 1, R = D0 (k), Cc = D1 * T
// -- so a tiled transpose through shared memory serves them, with coalesced reads AND writes (a gather
// with one side strided moved a 32-byte sector per 2-byte element).  Two kernels by the width of the
// source rows:
//   repack_weight_tile_kernel  Cc > 64: 64 x 64 tiles, two elements per thread on both sides.
//                              grid (ceil(Cc/64), ceil(Rp/64), B), 256 threads.
//   repack_weight_rows_kernel  Cc <= 64 (the taps of one kernel): 64 source rows are one contiguous run of
//                              64 * Cc elements, read linearly.  grid (ceil(Rp/64), B), 256 threads.
__device__ __forceinline__ void store_enc2(int enc, void* out0, void* out1, size_t i, float a, float b) {
    if (enc == ENC_F16) {
        *reinterpret_cast<__half2*>(reinterpret_cast<__half*>(out0) + i) = __floats2half2_rn(a, b);  // i is even
    } else {
        store_enc(enc, out0, out1, i, a);
        store_enc(enc, out0, out1, i + 1, b);
    }
}

template <typename TIn>
__global__ void __launch_bounds__(256) repack_weight_tile_kernel(const TIn* __restrict__ w, void* out0, void* out1, int enc,
                                                                 int R, int Cc, int Rp) {
    __shared__ float tile[64][65];  // [r][c]
    const int c0 = blockIdx.x * 64, r0 = blockIdx.y * 64;
    const size_t b = blockIdx.z;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    for (int j = ty; j < 64; j += 8) {
        const int r = r0 + j, c = c0 + 2 * tx;
        const size_t src = (b * R + r) * Cc + c;
        tile[j][2 * tx] = (r < R && c < Cc) ? load_as_float(w, src) : 0.f;
        tile[j][2 * tx + 1] = (r < R && c + 1 < Cc) ? load_as_float(w, src + 1) : 0.f;
    }
    __syncthreads();
    for (int j = ty; j < 64; j += 8) {
        const int c = c0 + j, r = r0 + 2 * tx;  // Rp is a multiple of the K block, so r + 1 < Rp whenever r < Rp
        if (c < Cc && r < Rp) store_enc2(enc, out0, out1, (b * Cc + c) * Rp + r, tile[2 * tx][j], tile[2 * tx + 1][j]);
    }
}

template <typename TIn>
__global__ void __launch_bounds__(256) repack_weight_rows_kernel(const TIn* __restrict__ w, void* out0, void* out1, int enc,
                                                                 int R, int Cc, int Rp) {
    __shared__ float tile[64][65];  // [c][r]
    const int r0 = blockIdx.x * 64;
    const size_t b = blockIdx.y;
    const int rows = min(64, R - r0);  // may be <= 0: a block of pure padding
    const int n_valid = rows > 0 ? rows * Cc : 0;
    const size_t base = (b * R + r0) * Cc;
    for (int i = threadIdx.x; i < 64 * Cc; i += 256) {
        const int r = i / Cc, c = i - r * Cc;
        tile[c][r] = (i < n_valid) ? load_as_float(w, base + i) : 0.f;
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < Cc * 32; idx += 256) {
        const int c = idx >> 5, r = (idx & 31) * 2;
        if (r0 + r < Rp) store_enc2(enc, out0, out1, (b * Cc + c) * Rp + r0 + r, tile[c][r], tile[c][r + 1]);
    }
}

// Few-channel activations (C <= 8, e.g. RGB stems): copy into a zero-padded NHWC image with exactly 8
// fp16 channels per pixel, [N][Hp][Wp][8], the original at offset (pad_h, pad_w).  One thread per
// padded pixel, one 16-byte store each.  A row of 8 consecutive pixels of this image is one 128-byte
// K slice holding (kw, c) for 8 taps, which is what the small-channel contraction path reads.
template <typename TIn>
__global__ void __launch_bounds__(256) pad_pack_c8_kernel(const TIn* __restrict__ in, int nchw, __half* __restrict__ out,
                                                          int N, int C, int H, int W, int pad_h, int pad_w, int Hp,
                                                          int Wp, float* colsum) {
    const size_t total = static_cast<size_t>(N) * Hp * Wp;
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};  // per-channel sums of the values read (bias gradient)
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int wp = static_cast<int>(i % Wp);
        const size_t r = i / Wp;
        const int hp = static_cast<int>(r % Hp);
        const int n = static_cast<int>(r / Hp);
        const int h = hp - pad_h, w = wp - pad_w;
        __half v[8];
#pragma unroll
        for (int c = 0; c < 8; ++c) v[c] = __float2half_rn(0.f);
        if (h >= 0 && h < H && w >= 0 && w < W) {
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                if (c < C) {
                    size_t src = nchw ? ((static_cast<size_t>(n) * C + c) * H + h) * W + w
                                      : ((static_cast<size_t>(n) * H + h) * W + w) * C + c;
                    const float xv = load_as_float(in, src);
                    v[c] = __float2half_rn(xv);
                    acc[c] += xv;  // the bias gradient sums the values as given, like every other column-sum path
                }
            }
        }
        reinterpret_cast<uint4*>(out)[i] = *reinterpret_cast<const uint4*>(v);
    }
    if (colsum != nullptr) {  // uniform across the grid
        __shared__ float part[8][8];
        const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
            float x = acc[c];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
            if (lane == 0) part[wy][c] = x;
        }
        __syncthreads();
        if (threadIdx.x < 8) {  // row blockIdx.x of the [blocks][8] partial-sum matrix
            float sum = 0.f;
#pragma unroll
            for (int w8 = 0; w8 < 8; ++w8) sum += part[w8][threadIdx.x];
            colsum[static_cast<size_t>(blockIdx.x) * 8 + threadIdx.x] = sum;
        }
    }
}

// Weights [C_out][C][KH][KW] -> [C_out][KH][64] with k = kw*8 + c (zero where c >= C or kw >= KW):
// the K-major operand matching pad_pack_c8's (kw, c) slices.
template <typename TIn>
__global__ void __launch_bounds__(256) repack_weight_c8_kernel(const TIn* __restrict__ w, __half* __restrict__ out,
                                                               int Cout, int C, int KH, int KW) {
    const int total = Cout * KH * 64;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int k = i & 63;
        const int kh = (i >> 6) % KH;
        const int co = (i >> 6) / KH;
        const int kw = k >> 3, c = k & 7;
        float v = 0.f;
        if (c < C && kw < KW) v = load_as_float(w, ((static_cast<size_t>(co) * C + c) * KH + kh) * KW + kw);
        out[i] = __float2half_rn(v);
    }
}

// Partial sums of a K-split forward walk, `planes` fp32 planes of [pixels][C] (one per K slice) -> the
// output tensor: the planes are added in slice order (so the result is bitwise repeatable), then bias,
// optional rounding through fp16, cast, and the caller's layout (nchw: out[n][c][pixel of the image]).
template <typename TOut>
__global__ void __launch_bounds__(256) finish_rows_kernel(const float* __restrict__ acc, int planes, const float* __restrict__ bias,
                                                          TOut* __restrict__ out, size_t pixels, int C, int hw, int nchw,
                                                          int round_f16) {
    const size_t total = pixels * C;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t p = i / C;
        const int c = static_cast<int>(i - p * C);
        float v = acc[i];
#pragma unroll 4
        for (int z = 1; z < planes; ++z) v += __ldg(acc + static_cast<size_t>(z) * total + i);
        if (bias != nullptr) v += bias[c];
        if (round_f16) v = __half2float(__float2half_rn(v));
        size_t o = i;
        if (nchw) {
            const size_t n = p / hw;
            o = (n * C + c) * hw + (p - n * hw);
        }
        out[o] = static_cast<TOut>(v);
    }
}

// Phase-packed gather walk: the weights [K][C][KH][KW] of a strided gather (input gradient of a
// convolution, forward of a transposed one; unit dilation) as the weights [N'][K][KH'][KW'] of the
// unit-stride convolution that computes all stride_h x stride_w output phases at once:
// n' = (ph * s_w + pw) * C + c, tap (kh', kw') reads the input at offset (kh' + dh_min, kw' + dw_min),
// which phase ph reaches through kernel row kh = ph + p_h - (kh' + dh_min) * s_h (zero weight if that
// is no kernel row).  Also replicates the bias per phase.
template <typename TIn, typename TBias>
__global__ void __launch_bounds__(256) pack_phase_weights_kernel(const TIn* __restrict__ w, __half* __restrict__ out,
                                                                 const TBias* __restrict__ bias, float* __restrict__ bias_out,
                                                                 int K, int C, int KH, int KW, int s_h, int s_w, int p_h,
                                                                 int p_w, int khp, int kwp, int dh_min, int dw_min) {
    const int np = s_h * s_w * C;
    const int total = np * K * khp * kwp;
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < total; i += gridDim.x * blockDim.x) {
        const int kw2 = i % kwp;
        int r = i / kwp;
        const int kh2 = r % khp;
        r /= khp;
        const int k = r % K;
        const int n2 = r / K;
        const int c = n2 % C;
        const int pw = (n2 / C) % s_w;
        const int ph = n2 / (C * s_w);
        const int kh = ph + p_h - (kh2 + dh_min) * s_h;
        const int kw = pw + p_w - (kw2 + dw_min) * s_w;
        float v = 0.f;
        if (kh >= 0 && kh < KH && kw >= 0 && kw < KW)
            v = load_as_float(w, ((static_cast<size_t>(k) * C + c) * KH + kh) * KW + kw);
        out[i] = __float2half_rn(v);
    }
    if (bias_out != nullptr && blockIdx.x == 0 && threadIdx.x < np)
        bias_out[threadIdx.x] = (bias != nullptr) ? load_as_float(bias, threadIdx.x % C) : 0.f;
}

// Second stage of the column sums: adds rows [blockIdx.y * rows_per_block, ...) of the [P][stride]
// partial-sum matrix in a fixed order (eight interleaved running sums, then those eight in order) and
// writes row blockIdx.y of `out` ([segments][out_stride]).  Launched again on its own output while more
// than one segment is left.  blockDim = (32, 8).
__global__ void __launch_bounds__(256) colsum_finish_kernel(const float* __restrict__ partial, int P, int stride, int C,
                                                            float* __restrict__ out, int out_stride, int rows_per_block) {
    __shared__ float part[8][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    const int p0 = blockIdx.y * rows_per_block;
    const int p1 = min(P, p0 + rows_per_block);
    float s = 0.f;
    if (c < C) {
#pragma unroll 4
        for (int p = p0 + threadIdx.y; p < p1; p += 8) s += __ldg(partial + static_cast<size_t>(p) * stride + c);
    }
    part[threadIdx.y][threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        float t = 0.f;
#pragma unroll
        for (int k = 0; k < 8; ++k) t += part[k][threadIdx.x];
        out[static_cast<size_t>(blockIdx.y) * out_stride + c] = t;
    }
}

// Second stage of a split-K weight gradient: adds the K slices' planes in slice order (bitwise
// repeatable, unlike atomics) and writes dW once.  Row form: dW is `rows` rows of `row_len4` float4,
// plane z holds row r at planes + z * plane_elems + r * src_pitch (floats).
__global__ void __launch_bounds__(256) wgrad_reduce_rows4_kernel(const float* __restrict__ planes, float* __restrict__ dw,
                                                                 int split, size_t plane_elems, size_t rows, int row_len4,
                                                                 size_t src_pitch) {
    const size_t total = rows * row_len4;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const size_t r = i / row_len4;
        const int c4 = static_cast<int>(i - r * row_len4);
        const float4* src = reinterpret_cast<const float4*>(planes + r * src_pitch) + c4;
        float4 a = __ldg(src);
        const size_t step = plane_elems / 4;
#pragma unroll 4
        for (int z = 1; z < split; ++z) {
            const float4 b = __ldg(src + z * step);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
        reinterpret_cast<float4*>(dw)[i] = a;
    }
}

// The same for many planes over a small gradient (the patch walk cuts K into one slice per SM): a thread
// per element would walk ~150 planes one load latency at a time.  blockDim = (32, 8): lane ty adds
// planes ty, ty + 8, ... of its float4 in order, then the eight running sums are added in order -- a
// fixed association, so still bitwise repeatable.  Planes are laid out like dW.
__global__ void __launch_bounds__(256) wgrad_reduce_deep4_kernel(const float* __restrict__ planes, float* __restrict__ dw,
                                                                 int split, size_t plane_elems, size_t total4) {
    __shared__ float4 part[8][32];
    const size_t i = blockIdx.x * 32ull + threadIdx.x;
    float4 a = make_float4(0.f, 0.f, 0.f, 0.f);
    if (i < total4) {
        const float4* src = reinterpret_cast<const float4*>(planes) + i;
        const size_t step = plane_elems / 4;
#pragma unroll 4
        for (int z = threadIdx.y; z < split; z += 8) {
            const float4 b = __ldg(src + z * step);
            a.x += b.x; a.y += b.y; a.z += b.z; a.w += b.w;
        }
    }
    part[threadIdx.y][threadIdx.x] = a;
    __syncthreads();
    if (threadIdx.y == 0 && i < total4) {
        float4 t = part[0][threadIdx.x];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
            const float4 b = part[k][threadIdx.x];
            t.x += b.x; t.y += b.y; t.z += b.z; t.w += b.w;
        }
        reinterpret_cast<float4*>(dw)[i] = t;
    }
}

// General form, one thread per dW element.  layout 0: a plane is laid out like dW.  layout 1: a plane is
// [plain channel][R rows of the tile walk] and dW element (plain, pc, t) sits at row
// (t * c_blocks + pc / kb) * kb + pc % kb.  layout 2 (few-channel window walk): dW element
// (plain, c, kh, kw) sits at row kh * kb + kw * 8 + c.
__global__ void __launch_bounds__(256) wgrad_reduce_kernel(const float* __restrict__ planes, float* __restrict__ dw, int split,
                                                           size_t plane_elems, size_t total, int layout, int c_patch,
                                                           int n_taps, int kw_count, int c_blocks, int kb, int R) {
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total;
         i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        size_t src = i;
        if (layout == 1) {
            const int t = static_cast<int>(i % n_taps);
            const size_t q = i / n_taps;
            const int pc = static_cast<int>(q % c_patch);
            const size_t plain = q / c_patch;
            src = plain * R + static_cast<size_t>(t * c_blocks + pc / kb) * kb + pc % kb;
        } else if (layout == 2) {
            const int kw = static_cast<int>(i % kw_count);
            size_t q = i / kw_count;
            const int kh = static_cast<int>(q % n_taps);
            q /= n_taps;
            const int c = static_cast<int>(q % c_patch);
            const size_t plain = q / c_patch;
            src = plain * R + static_cast<size_t>(kh) * kb + kw * 8 + c;
        }
        float a = __ldg(planes + src);
        for (int z = 1; z < split; ++z) a += __ldg(planes + z * plane_elems + src);
        dw[i] = a;
    }
}

template <typename TIn>
__global__ void __launch_bounds__(256) to_float_kernel(const TIn* __restrict__ in, float* out, int n) {
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = load_as_float(in, i);
}

}  // namespace nml
