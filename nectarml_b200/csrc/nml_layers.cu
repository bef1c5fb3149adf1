// Memory-bound neighbours of the contraction path in a training step, on the layout the contraction
// kernels keep between layers (fp16 NHWC, i.e. a row-major [pixels][channels] matrix):
//   * batch normalisation fused with the activation and the residual add that follow it, forward and
//     backward (replaces the reference's fp32-NCHW Welford / normalize / backward kernels,
//     nectarml/csrc/kernels/tensor/fused/norm.cu, and the separate ReLU / LeakyReLU / add passes
//     around them);
//   * one unscale + finiteness check and one SGD-momentum update over a FLAT parameter buffer
//     (replaces one unscale launch + cudaMalloc + blocking read-back per parameter,
//     nectarml/csrc/ops/amp/amp.cpp:18-37, and one update launch per parameter,
//     nectarml/optim/sgd.py:75-90, nectarml/csrc/kernels/optim/sgd.cu).
// Every reduction is two-stage with a fixed order (no atomics): results are bitwise repeatable.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <atomic>

#include "../../include/nectarml_b200.h"

namespace nml_layers {

#define NMLL_CUDA(expr)                              \
    do {                                             \
        cudaError_t e_ = (expr);                     \
        if (e_ != cudaSuccess) return NML_ERR_CUDA;  \
    } while (0)

static inline size_t round_up(size_t v, size_t m) { return (v + m - 1) / m * m; }
static std::atomic<long long> g_layer_launches{0};

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const float2 t = __half22float2(h[j]);
        f[2 * j] = t.x;
        f[2 * j + 1] = t.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __half2* h = reinterpret_cast<__half2*>(&v);
#pragma unroll
    for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
    return v;
}
// derivative of the activation, read off the activation's OUTPUT: 0 none, 1 ReLU, 2 LeakyReLU(slope)
__device__ __forceinline__ float act_grad(int act, float slope, float y) {
    return act == 0 ? 1.f : (y > 0.f ? 1.f : (act == 1 ? 0.f : slope));
}

// Thread layout shared by the kernels below: the matrix is [M][C] fp16 with C a multiple of 8, a
// vector is 8 adjacent channels (16 bytes), cpr = C / 8 vectors per row.  A block has
// (256 / cpr) * cpr threads; thread t owns vector column t % cpr for good (its per-channel
// constants sit in registers) and walks rows t / cpr, + rows-per-pass, ...: consecutive threads read
// consecutive 16-byte vectors, so every access is fully coalesced whatever C is.

// First stage of a per-channel reduction over rows.  kBackward == false: a = sum x, b = sum x^2.
// kBackward == true: with dz = dy * act'(y): a = sum dz, b = sum dz * x (the second stage turns b into
// d gamma = rstd * (b - mean * a), so this pass needs no per-channel constants).  Two rows are in flight
// per thread.  Block p writes its sums to partial[p][0..C) and partial[p][C..2C).
template <bool kBackward>
__global__ void __launch_bounds__(256) bn_reduce_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy,
                                                        const uint4* __restrict__ y, int act, float slope,
                                                        float* __restrict__ partial, size_t M, int C) {
    __shared__ float sm[256][17];
    const int cpr = C >> 3;
    const int rpb = blockDim.x / cpr;
    const int col = threadIdx.x % cpr, rsub = threadIdx.x / cpr;
    float a[8], b[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) a[j] = b[j] = 0.f;
    auto add = [&](const uint4& xv, const uint4& dv, const uint4& yv) {
        float xf[8];
        unpack8(xv, xf);
        if (!kBackward) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                a[j] += xf[j];
                b[j] += xf[j] * xf[j];
            }
        } else {
            float df[8], yf[8];
            unpack8(dv, df);
            if (act != 0) unpack8(yv, yf);
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float dz = df[j] * (act != 0 ? act_grad(act, slope, yf[j]) : 1.f);
                a[j] += dz;
                b[j] += dz * xf[j];
            }
        }
    };
    const size_t stride = static_cast<size_t>(gridDim.x) * rpb;
    size_t row = static_cast<size_t>(blockIdx.x) * rpb + rsub;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    if (!kBackward) {  // one input stream only: four rows in flight keep as many bytes outstanding as the backward pass has
        for (; row + 3 * stride < M; row += 4 * stride) {
            const uint4 x0 = __ldg(x + row * cpr + col), x1 = __ldg(x + (row + stride) * cpr + col);
            const uint4 x2 = __ldg(x + (row + 2 * stride) * cpr + col), x3 = __ldg(x + (row + 3 * stride) * cpr + col);
            add(x0, zero, zero);
            add(x1, zero, zero);
            add(x2, zero, zero);
            add(x3, zero, zero);
        }
    }
    for (; row + stride < M; row += 2 * stride) {
        const size_t v0 = row * cpr + col, v1 = (row + stride) * cpr + col;
        const uint4 x0 = __ldg(x + v0), x1 = __ldg(x + v1);
        const uint4 d0 = kBackward ? __ldg(dy + v0) : zero, d1 = kBackward ? __ldg(dy + v1) : zero;
        const uint4 y0 = (kBackward && act != 0) ? __ldg(y + v0) : zero, y1 = (kBackward && act != 0) ? __ldg(y + v1) : zero;
        add(x0, d0, y0);
        add(x1, d1, y1);
    }
    if (row < M) {
        const size_t v0 = row * cpr + col;
        add(__ldg(x + v0), kBackward ? __ldg(dy + v0) : zero, (kBackward && act != 0) ? __ldg(y + v0) : zero);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        sm[threadIdx.x][j] = a[j];
        sm[threadIdx.x][8 + j] = b[j];
    }
    __syncthreads();
    if (threadIdx.x < cpr) {  // fixed order over the block's row lanes
        float* out = partial + static_cast<size_t>(blockIdx.x) * 2 * C;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float sa = 0.f, sb = 0.f;
            for (int r = 0; r < rpb; ++r) {
                sa += sm[r * cpr + threadIdx.x][j];
                sb += sm[r * cpr + threadIdx.x][8 + j];
            }
            out[threadIdx.x * 8 + j] = sa;
            out[C + threadIdx.x * 8 + j] = sb;
        }
    }
}

// Second stage: adds the P rows of partial sums in a fixed order (32 interleaved running sums in double,
// then those 32 in order).  mode 0: out0 = mean, out1 = 1 / sqrt(biased variance + eps).
// mode 1: out0 = sum a (d beta), out1 = rstd * (sum b - mean * sum a) (d gamma).  blockDim = (32, 32): the
// pass is a chain of load latencies, so it is spread over as many threads as a block has.
__global__ void __launch_bounds__(1024) bn_finish_kernel(const float* __restrict__ partial, int P, int C, int mode, double inv_M,
                                                        float eps, const float* __restrict__ mean, const float* __restrict__ rstd,
                                                        float* __restrict__ out0, float* __restrict__ out1) {
    __shared__ double pa[32][33], pb[32][33];
    const int c = blockIdx.x * 32 + threadIdx.x;
    double sa = 0.0, sb = 0.0;
    if (c < C) {
#pragma unroll 4
        for (int p = threadIdx.y; p < P; p += 32) {
            sa += static_cast<double>(__ldg(partial + static_cast<size_t>(p) * 2 * C + c));
            sb += static_cast<double>(__ldg(partial + static_cast<size_t>(p) * 2 * C + C + c));
        }
    }
    pa[threadIdx.y][threadIdx.x] = sa;
    pb[threadIdx.y][threadIdx.x] = sb;
    __syncthreads();
    if (threadIdx.y == 0 && c < C) {
        double ta = 0.0, tb = 0.0;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            ta += pa[k][threadIdx.x];
            tb += pb[k][threadIdx.x];
        }
        if (mode == 0) {
            const double m = ta * inv_M;
            double var = tb * inv_M - m * m;
            if (var < 0.0) var = 0.0;
            out0[c] = static_cast<float>(m);
            out1[c] = static_cast<float>(1.0 / sqrt(var + static_cast<double>(eps)));
        } else {
            out0[c] = static_cast<float>(ta);
            out1[c] = static_cast<float>(static_cast<double>(rstd[c]) * (tb - static_cast<double>(mean[c]) * ta));
        }
    }
}

// y = act(gamma * (x - mean) * rstd + beta [+ residual]), fp16 in and out; two rows in flight per thread.
__global__ void __launch_bounds__(256) bn_apply_kernel(const uint4* __restrict__ x, const uint4* __restrict__ res,
                                                       uint4* __restrict__ y, const float* __restrict__ gamma,
                                                       const float* __restrict__ beta, const float* __restrict__ mean,
                                                       const float* __restrict__ rstd, int act, float slope, size_t M, int C) {
    const int cpr = C >> 3;
    const int rpb = blockDim.x / cpr;
    const int col = threadIdx.x % cpr, rsub = threadIdx.x / cpr;
    float sc[8], sh[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = col * 8 + j;
        sc[j] = (gamma ? gamma[c] : 1.f) * rstd[c];
        sh[j] = (beta ? beta[c] : 0.f) - mean[c] * sc[j];
    }
    auto one = [&](const uint4& xv, const uint4& rv) -> uint4 {
        float xf[8], rf[8];
        unpack8(xv, xf);
        if (res) unpack8(rv, rf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            float t = xf[j] * sc[j] + sh[j];
            if (res) t += rf[j];
            if (act != 0 && t < 0.f) t = (act == 1) ? 0.f : t * slope;
            xf[j] = t;
        }
        return pack8(xf);
    };
    const size_t stride = static_cast<size_t>(gridDim.x) * rpb;
    size_t row = static_cast<size_t>(blockIdx.x) * rpb + rsub;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (; row + stride < M; row += 2 * stride) {
        const size_t v0 = row * cpr + col, v1 = (row + stride) * cpr + col;
        const uint4 x0 = __ldg(x + v0), x1 = __ldg(x + v1);
        const uint4 r0 = res ? __ldg(res + v0) : zero, r1 = res ? __ldg(res + v1) : zero;
        y[v0] = one(x0, r0);
        y[v1] = one(x1, r1);
    }
    if (row < M) {
        const size_t v0 = row * cpr + col;
        y[v0] = one(__ldg(x + v0), res ? __ldg(res + v0) : zero);
    }
}

// dx = gamma * rstd * (dz - dbeta / M - xhat * dgamma / M) with dz = dy * act'(y), folded into
// dx = A * dz + B * x + C per channel; optionally dres = dz (the gradient of the residual input that was
// added before the activation).  Two rows in flight per thread.
__global__ void __launch_bounds__(256) bn_dx_kernel(const uint4* __restrict__ x, const uint4* __restrict__ dy,
                                                    const uint4* __restrict__ y, uint4* __restrict__ dx, uint4* __restrict__ dres,
                                                    const float* __restrict__ gamma, const float* __restrict__ mean,
                                                    const float* __restrict__ rstd, const float* __restrict__ dbeta,
                                                    const float* __restrict__ dgamma, int act, float slope, float inv_M,
                                                    size_t M, int C) {
    const int cpr = C >> 3;
    const int rpb = blockDim.x / cpr;
    const int col = threadIdx.x % cpr, rsub = threadIdx.x / cpr;
    float ka[8], kb[8], kc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        const int c = col * 8 + j;
        const float rs = rstd[c], mu = mean[c];
        const float k0 = (gamma ? gamma[c] : 1.f) * rs, k1 = dbeta[c] * inv_M, k2 = dgamma[c] * inv_M;
        ka[j] = k0;
        kb[j] = -k0 * rs * k2;
        kc[j] = k0 * (mu * rs * k2 - k1);
    }
    auto one = [&](const uint4& xv, const uint4& dv, const uint4& yv, uint4& dz_out) -> uint4 {
        float xf[8], df[8], yf[8];
        unpack8(xv, xf);
        unpack8(dv, df);
        if (act != 0) unpack8(yv, yf);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float dz = df[j] * (act != 0 ? act_grad(act, slope, yf[j]) : 1.f);
            df[j] = dz;
            xf[j] = ka[j] * dz + kb[j] * xf[j] + kc[j];
        }
        dz_out = pack8(df);
        return pack8(xf);
    };
    const size_t stride = static_cast<size_t>(gridDim.x) * rpb;
    size_t row = static_cast<size_t>(blockIdx.x) * rpb + rsub;
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
    for (; row + stride < M; row += 2 * stride) {
        const size_t v0 = row * cpr + col, v1 = (row + stride) * cpr + col;
        const uint4 x0 = __ldg(x + v0), x1 = __ldg(x + v1), d0 = __ldg(dy + v0), d1 = __ldg(dy + v1);
        const uint4 y0 = act != 0 ? __ldg(y + v0) : zero, y1 = act != 0 ? __ldg(y + v1) : zero;
        uint4 z0, z1;
        dx[v0] = one(x0, d0, y0, z0);
        dx[v1] = one(x1, d1, y1, z1);
        if (dres) {
            dres[v0] = z0;
            dres[v1] = z1;
        }
    }
    if (row < M) {
        const size_t v0 = row * cpr + col;
        uint4 z0;
        dx[v0] = one(__ldg(x + v0), __ldg(dy + v0), act != 0 ? __ldg(y + v0) : zero, z0);
        if (dres) dres[v0] = z0;
    }
}

// any(!isfinite(g * inv_scale)) over a flat fp32 buffer -> *found (set, never cleared, here)
__global__ void __launch_bounds__(256) grads_check_kernel(const float4* __restrict__ g, size_t n4, float inv_scale, int* found) {
    bool bad = false;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const float4 v = __ldg(g + i);
        bad |= !isfinite(v.x * inv_scale) | !isfinite(v.y * inv_scale) | !isfinite(v.z * inv_scale) | !isfinite(v.w * inv_scale);
    }
    if (__any_sync(0xffffffffu, bad) && (threadIdx.x & 31) == 0) *found = 1;  // every writer writes the same value
}

// One SGD-momentum update over the whole flat buffer: g = grad * inv_scale + wd * p; v = momentum * v +
// (1 - dampening) * g; p -= lr * v; and the fp16 copy of p the next forward reads.  Skipped as a whole
// when *found_inf is set (the GradScaler rule: an overflowed step leaves the parameters alone).
__global__ void __launch_bounds__(256) sgd_momentum_kernel(float4* __restrict__ p, const float4* __restrict__ g, float4* __restrict__ vel,
                                                           uint2* __restrict__ p16, size_t n4, float lr, float momentum, float dampening,
                                                           float wd, float inv_scale, const int* __restrict__ found_inf) {
    if (found_inf && *found_inf) return;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < n4; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        float4 pv = p[i], vv = vel[i];
        const float4 gv = __ldg(g + i);
        float* pp = reinterpret_cast<float*>(&pv);
        float* vp = reinterpret_cast<float*>(&vv);
        const float* gp = reinterpret_cast<const float*>(&gv);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const float gg = gp[j] * inv_scale + wd * pp[j];
            vp[j] = momentum * vp[j] + (1.f - dampening) * gg;
            pp[j] -= lr * vp[j];
        }
        p[i] = pv;
        vel[i] = vv;
        if (p16) {
            uint2 h;
            *reinterpret_cast<__half2*>(&h.x) = __floats2half2_rn(pp[0], pp[1]);
            *reinterpret_cast<__half2*>(&h.y) = __floats2half2_rn(pp[2], pp[3]);
            p16[i] = h;
        }
    }
}

// Max pooling over NHWC fp16, 8 channels per thread.  Forward also records, per output value, which tap of
// the window won (kh * k + kw, one byte); backward is a GATHER over the <= ceil(k/s)^2 windows that cover an
// input pixel -- no atomics, so it is bitwise repeatable, and every input gradient is written exactly once
// (no zero-fill pass).  Out-of-image taps are skipped (i.e. padded with -inf).
__global__ void __launch_bounds__(256) maxpool_fwd_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, uint2* __restrict__ idx,
                                                          int N, int H, int W, int C, int k, int s, int p, int Ho, int Wo) {
    const int cpr = C >> 3;
    const size_t total = static_cast<size_t>(N) * Ho * Wo * cpr;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int cv = static_cast<int>(i % cpr);
        size_t r = i / cpr;
        const int ow = static_cast<int>(r % Wo);
        r /= Wo;
        const int oh = static_cast<int>(r % Ho);
        const int n = static_cast<int>(r / Ho);
        float best[8];
        unsigned char who[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            best[j] = -INFINITY;
            who[j] = 0;
        }
        for (int kh = 0; kh < k; ++kh) {
            const int ih = oh * s - p + kh;
            if (ih < 0 || ih >= H) continue;
            for (int kw = 0; kw < k; ++kw) {
                const int iw = ow * s - p + kw;
                if (iw < 0 || iw >= W) continue;
                float f[8];
                unpack8(__ldg(x + ((static_cast<size_t>(n) * H + ih) * W + iw) * cpr + cv), f);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    if (f[j] > best[j]) {
                        best[j] = f[j];
                        who[j] = static_cast<unsigned char>(kh * k + kw);
                    }
            }
        }
        y[i] = pack8(best);
        uint2 w2;
        w2.x = who[0] | (who[1] << 8) | (who[2] << 16) | (who[3] << 24);
        w2.y = who[4] | (who[5] << 8) | (who[6] << 16) | (who[7] << 24);
        idx[i] = w2;
    }
}

__global__ void __launch_bounds__(256) maxpool_bwd_kernel(const uint4* __restrict__ dy, const uint2* __restrict__ idx, uint4* __restrict__ dx,
                                                          int N, int H, int W, int C, int k, int s, int p, int Ho, int Wo) {
    const int cpr = C >> 3;
    const size_t total = static_cast<size_t>(N) * H * W * cpr;
    for (size_t i = blockIdx.x * static_cast<size_t>(blockDim.x) + threadIdx.x; i < total; i += static_cast<size_t>(gridDim.x) * blockDim.x) {
        const int cv = static_cast<int>(i % cpr);
        size_t r = i / cpr;
        const int iw = static_cast<int>(r % W);
        r /= W;
        const int ih = static_cast<int>(r % H);
        const int n = static_cast<int>(r / H);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        // windows (oh, ow) with 0 <= ih + p - oh * s < k
        const int oh_hi = min((ih + p) / s, Ho - 1), ow_hi = min((iw + p) / s, Wo - 1);
        for (int oh = oh_hi; oh >= 0 && ih + p - oh * s < k; --oh) {
            const int kh = ih + p - oh * s;
            for (int ow = ow_hi; ow >= 0 && iw + p - ow * s < k; --ow) {
                const int me = kh * k + (iw + p - ow * s);
                const size_t o = ((static_cast<size_t>(n) * Ho + oh) * Wo + ow) * cpr + cv;
                const uint2 w2 = __ldg(idx + o);
                float g[8];
                unpack8(__ldg(dy + o), g);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    const unsigned who = ((j < 4 ? w2.x : w2.y) >> (8 * (j & 3))) & 0xffu;
                    if (who == static_cast<unsigned>(me)) acc[j] += g[j];
                }
            }
        }
        dx[i] = pack8(acc);
    }
}

static int bn_grid(long long M, int C, int* threads) {
    const int cpr = C / 8;
    *threads = (256 / cpr) * cpr;
    const int rpb = *threads / cpr;
    const long long want = (M + rpb - 1) / rpb;
    return static_cast<int>(want < 148 * 4 ? want : 148 * 4);
}
static int bn_grid_elementwise(long long M, int C) {  // no partial sums behind these: as many blocks as keep HBM busy
    const int cpr = C / 8;
    const int rpb = ((256 / cpr) * cpr) / cpr;
    const long long want = (M + rpb - 1) / rpb;
    return static_cast<int>(want < 148 * 16 ? want : 148 * 16);
}
static bool bn_shape_ok(long long M, int C) { return M > 0 && C > 0 && C % 8 == 0 && C <= 2048; }
static bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

}  // namespace nml_layers

using namespace nml_layers;

extern "C" {

int nml_bn_workspace_size(long long rows, int channels, size_t* bytes) {
    if (!bytes || !bn_shape_ok(rows, channels)) return NML_ERR_INVALID;
    int threads;
    const int P = bn_grid(rows, channels, &threads);
    *bytes = round_up(static_cast<size_t>(P) * 2 * channels * sizeof(float), 256);
    return NML_OK;
}

int nml_bn_forward(const void* x, long long rows, int channels, const float* gamma, const float* beta, const void* residual,
                   int act, float slope, float eps, void* y, float* mean, float* rstd, void* workspace,
                   size_t workspace_bytes, void* stream) {
    if (!x || !y || !mean || !rstd || act < 0 || act > 2) return NML_ERR_INVALID;
    if (!bn_shape_ok(rows, channels)) return NML_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(y) || (residual && !aligned16(residual))) return NML_ERR_INVALID;
    size_t need = 0;
    nml_bn_workspace_size(rows, channels, &need);
    if (!workspace || workspace_bytes < need) return NML_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int threads;
    const int P = bn_grid(rows, channels, &threads);
    float* partial = static_cast<float*>(workspace);
    bn_reduce_kernel<false><<<P, threads, 0, st>>>(static_cast<const uint4*>(x), nullptr, nullptr, 0, 0.f, partial,
                                                   static_cast<size_t>(rows), channels);
    bn_finish_kernel<<<(channels + 31) / 32, dim3(32, 32), 0, st>>>(partial, P, channels, 0, 1.0 / static_cast<double>(rows), eps,
                                                                   nullptr, nullptr, mean, rstd);
    bn_apply_kernel<<<bn_grid_elementwise(rows, channels), threads, 0, st>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(residual),
                                           static_cast<uint4*>(y), gamma, beta, mean, rstd, act, slope,
                                           static_cast<size_t>(rows), channels);
    NMLL_CUDA(cudaGetLastError());
    g_layer_launches += 3;
    return NML_OK;
}

int nml_bn_backward(const void* dy, const void* y, const void* x, long long rows, int channels, const float* gamma,
                    const float* mean, const float* rstd, int act, float slope, void* dx, void* dres, float* dgamma,
                    float* dbeta, void* workspace, size_t workspace_bytes, void* stream) {
    if (!dy || !x || !mean || !rstd || !dx || !dgamma || !dbeta || act < 0 || act > 2 || (act != 0 && !y)) return NML_ERR_INVALID;
    if (!bn_shape_ok(rows, channels)) return NML_ERR_UNSUPPORTED;
    if (!aligned16(dy) || !aligned16(x) || !aligned16(dx) || (y && !aligned16(y)) || (dres && !aligned16(dres))) return NML_ERR_INVALID;
    size_t need = 0;
    nml_bn_workspace_size(rows, channels, &need);
    if (!workspace || workspace_bytes < need) return NML_ERR_WORKSPACE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int threads;
    const int P = bn_grid(rows, channels, &threads);
    float* partial = static_cast<float*>(workspace);
    bn_reduce_kernel<true><<<P, threads, 0, st>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(dy),
                                                  static_cast<const uint4*>(y), act, slope, partial,
                                                  static_cast<size_t>(rows), channels);
    bn_finish_kernel<<<(channels + 31) / 32, dim3(32, 32), 0, st>>>(partial, P, channels, 1, 0.0, 0.f, mean, rstd, dbeta, dgamma);
    bn_dx_kernel<<<bn_grid_elementwise(rows, channels), threads, 0, st>>>(static_cast<const uint4*>(x), static_cast<const uint4*>(dy), static_cast<const uint4*>(y),
                                        static_cast<uint4*>(dx), static_cast<uint4*>(dres), gamma, mean, rstd, dbeta, dgamma, act,
                                        slope, static_cast<float>(1.0 / static_cast<double>(rows)), static_cast<size_t>(rows),
                                        channels);
    NMLL_CUDA(cudaGetLastError());
    g_layer_launches += 3;
    return NML_OK;
}

long long nml_layers_launch_count(void) { return g_layer_launches.load(); }

int nml_maxpool_forward(const void* x, int batch, int h, int w, int channels, int k, int stride, int pad, void* y,
                        void* index, void* stream) {
    if (!x || !y || !index || batch <= 0 || h <= 0 || w <= 0 || k <= 0 || k > 15 || stride <= 0 || pad < 0 || pad >= k)
        return NML_ERR_INVALID;
    if (channels <= 0 || channels % 8) return NML_ERR_UNSUPPORTED;
    if (!aligned16(x) || !aligned16(y) || (reinterpret_cast<uintptr_t>(index) & 7)) return NML_ERR_INVALID;
    const int ho = (h + 2 * pad - k) / stride + 1, wo = (w + 2 * pad - k) / stride + 1;
    if (ho <= 0 || wo <= 0) return NML_ERR_INVALID;
    const size_t total = static_cast<size_t>(batch) * ho * wo * (channels / 8);
    const int blocks = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    maxpool_fwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(x), static_cast<uint4*>(y),
                                                                             static_cast<uint2*>(index), batch, h, w, channels, k,
                                                                             stride, pad, ho, wo);
    NMLL_CUDA(cudaGetLastError());
    ++g_layer_launches;
    return NML_OK;
}

int nml_maxpool_backward(const void* dy, const void* index, int batch, int h, int w, int channels, int k, int stride, int pad,
                         void* dx, void* stream) {
    if (!dy || !dx || !index || batch <= 0 || h <= 0 || w <= 0 || k <= 0 || k > 15 || stride <= 0 || pad < 0 || pad >= k)
        return NML_ERR_INVALID;
    if (channels <= 0 || channels % 8) return NML_ERR_UNSUPPORTED;
    if (!aligned16(dy) || !aligned16(dx) || (reinterpret_cast<uintptr_t>(index) & 7)) return NML_ERR_INVALID;
    const int ho = (h + 2 * pad - k) / stride + 1, wo = (w + 2 * pad - k) / stride + 1;
    if (ho <= 0 || wo <= 0) return NML_ERR_INVALID;
    const size_t total = static_cast<size_t>(batch) * h * w * (channels / 8);
    const int blocks = static_cast<int>((total + 255) / 256 < 148 * 16 ? (total + 255) / 256 : 148 * 16);
    maxpool_bwd_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<const uint4*>(dy), static_cast<const uint2*>(index),
                                                                             static_cast<uint4*>(dx), batch, h, w, channels, k, stride,
                                                                             pad, ho, wo);
    NMLL_CUDA(cudaGetLastError());
    ++g_layer_launches;
    return NML_OK;
}

int nml_grads_check(const float* grads, size_t n, float inv_scale, int* found_inf, void* stream) {
    if (!grads || !found_inf || n % 4 || !aligned16(grads)) return NML_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    NMLL_CUDA(cudaMemsetAsync(found_inf, 0, sizeof(int), st));
    const size_t n4 = n / 4;
    const int blocks = static_cast<int>(n4 / 256 + 1 < 148 * 8 ? n4 / 256 + 1 : 148 * 8);
    grads_check_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<const float4*>(grads), n4, inv_scale, found_inf);
    NMLL_CUDA(cudaGetLastError());
    ++g_layer_launches;
    return NML_OK;
}

int nml_sgd_momentum_step(float* params, const float* grads, float* velocity, void* params_f16, size_t n, float lr,
                          float momentum, float dampening, float weight_decay, float inv_scale, const int* found_inf,
                          void* stream) {
    if (!params || !grads || !velocity || n % 4 || !aligned16(params) || !aligned16(grads) || !aligned16(velocity) ||
        (params_f16 && (reinterpret_cast<uintptr_t>(params_f16) & 7)))
        return NML_ERR_INVALID;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t n4 = n / 4;
    const int blocks = static_cast<int>(n4 / 256 + 1 < 148 * 8 ? n4 / 256 + 1 : 148 * 8);
    sgd_momentum_kernel<<<blocks, 256, 0, st>>>(reinterpret_cast<float4*>(params), reinterpret_cast<const float4*>(grads),
                                                reinterpret_cast<float4*>(velocity), static_cast<uint2*>(params_f16), n4, lr,
                                                momentum, dampening, weight_decay, inv_scale, found_inf);
    NMLL_CUDA(cudaGetLastError());
    ++g_layer_launches;
    return NML_OK;
}

}  // extern "C"
