/*
 * TEST INFRASTRUCTURE -- not part of the product.
 *
 * CPU restatement, in plain C, of the reference's NumPy backend for Conv2d / ConvTranspose2d
 * (nectarml/cpu/conv/conv2d.py in the reference project).  Only tests, the smoke check and the
 * CPU-baseline leg of the benchmark may call it; the CUDA library never does.
 *
 * Every function names the reference function it follows.  Loop nests keep the reference's
 * order and fp32 arithmetic (compile with -ffp-contract=off so products are rounded before
 * they are added, as NumPy float32 scalars are).  Where the reference hands an inner sum to
 * np.einsum / matmul, whose summation order is not specified, the sum here runs in index order.
 *
 * Pinned against outputs of the reference's own functions: tests/golden/ holds fixtures made
 * by importing the reference (tests/golden/make_golden.py).
 *
 * All tensors are dense fp32: activations NCHW, conv weight [C_out][C_in][KH][KW],
 * conv-transpose weight [C_in][C_out][KH][KW].  groups == 1.
 */
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#define IDX4(a, b, c, d, B_, C_, D_) ((((size_t)(a) * (B_) + (b)) * (C_) + (c)) * (D_) + (d))

/* _conv2d, nectarml/cpu/conv/conv2d.py:141-182.  Accumulates per output element starting from
 * the bias, over ci, then kh, then kw, reading zero where the padded input is zero. */
void nml_oracle_conv2d(const float* x, const float* w, const float* bias, float* y, int B, int C_in, int H, int W,
                       int C_out, int KH, int KW, int H_out, int W_out, int s_h, int s_w, int p_h, int p_w, int d_h,
                       int d_w) {
    for (int b = 0; b < B; ++b)
        for (int co = 0; co < C_out; ++co)
            for (int h = 0; h < H_out; ++h)
                for (int wo = 0; wo < W_out; ++wo) {
                    float s = bias ? bias[co] : 0.0f;
                    for (int ci = 0; ci < C_in; ++ci)
                        for (int kh = 0; kh < KH; ++kh) {
                            int ih = h * s_h + kh * d_h - p_h;
                            for (int kw = 0; kw < KW; ++kw) {
                                int iw = wo * s_w + kw * d_w - p_w;
                                float xv = (ih >= 0 && ih < H && iw >= 0 && iw < W) ? x[IDX4(b, ci, ih, iw, C_in, H, W)]
                                                                                     : 0.0f;
                                float prod = xv * w[IDX4(co, ci, kh, kw, C_in, KH, KW)];
                                s = s + prod;
                            }
                        }
                    y[IDX4(b, co, h, wo, C_out, H_out, W_out)] = s;
                }
}

/* _conv_transpose2d, nectarml/cpu/conv/conv2d.py:184-230.  Scatter into the full-size output
 * per (h, w, kh, kw) with a [B,C_in]x[C_in,C_out] product, crop the padding, add the bias. */
void nml_oracle_conv_transpose2d(const float* x, const float* w, const float* bias, float* y, int B, int C_in, int H,
                                 int W, int C_out, int KH, int KW, int s_h, int s_w, int p_h, int p_w, int d_h,
                                 int d_w, int op_h, int op_w) {
    int H_full = (H - 1) * s_h + d_h * (KH - 1) + 1;
    int W_full = (W - 1) * s_w + d_w * (KW - 1) + 1;
    int H_out = H_full - 2 * p_h + op_h;
    int W_out = W_full - 2 * p_w + op_w;
    /* the reference crops a [.., p : p + H_out] slice of the full buffer; rows past H_full do
     * not exist there, so give the full buffer room for the output padding and keep it zero */
    int Hf = H_full > p_h + H_out ? H_full : p_h + H_out;
    int Wf = W_full > p_w + W_out ? W_full : p_w + W_out;
    float* full = (float*)calloc((size_t)B * C_out * Hf * Wf, sizeof(float));
    for (int h = 0; h < H; ++h)
        for (int wi = 0; wi < W; ++wi)
            for (int kh = 0; kh < KH; ++kh)
                for (int kw = 0; kw < KW; ++kw) {
                    int oh = h * s_h + kh * d_h, ow = wi * s_w + kw * d_w;
                    for (int b = 0; b < B; ++b)
                        for (int co = 0; co < C_out; ++co) {
                            float acc = 0.0f;
                            for (int ci = 0; ci < C_in; ++ci) {
                                float prod = x[IDX4(b, ci, h, wi, C_in, H, W)] * w[IDX4(ci, co, kh, kw, C_out, KH, KW)];
                                acc = acc + prod;
                            }
                            full[IDX4(b, co, oh, ow, C_out, Hf, Wf)] += acc;
                        }
                }
    for (int b = 0; b < B; ++b)
        for (int co = 0; co < C_out; ++co)
            for (int h = 0; h < H_out; ++h)
                for (int wo = 0; wo < W_out; ++wo) {
                    float v = full[IDX4(b, co, h + p_h, wo + p_w, C_out, Hf, Wf)];
                    if (bias) v = v + bias[co];
                    y[IDX4(b, co, h, wo, C_out, H_out, W_out)] = v;
                }
    free(full);
}

/* _conv2d_backward_input, nectarml/cpu/conv/conv2d.py:232-278.  Per (h, w, kh, kw) adds
 * einsum('bo,oi->bi', dY[:,:,h,w], W[:,:,kh,kw]) into the padded gradient, then crops. */
void nml_oracle_conv2d_backward_input(const float* dy, const float* w, float* dx, int B, int C_in, int H, int W,
                                      int C_out, int KH, int KW, int H_out, int W_out, int s_h, int s_w, int p_h,
                                      int p_w, int d_h, int d_w) {
    int Hp = H + 2 * p_h, Wp = W + 2 * p_w;
    float* gp = (float*)calloc((size_t)B * C_in * Hp * Wp, sizeof(float));
    for (int h = 0; h < H_out; ++h)
        for (int wo = 0; wo < W_out; ++wo)
            for (int kh = 0; kh < KH; ++kh)
                for (int kw = 0; kw < KW; ++kw) {
                    int ih = h * s_h + kh * d_h, iw = wo * s_w + kw * d_w;
                    if (ih >= Hp || iw >= Wp) continue;
                    for (int b = 0; b < B; ++b)
                        for (int ci = 0; ci < C_in; ++ci) {
                            float acc = 0.0f;
                            for (int co = 0; co < C_out; ++co) {
                                float prod =
                                    dy[IDX4(b, co, h, wo, C_out, H_out, W_out)] * w[IDX4(co, ci, kh, kw, C_in, KH, KW)];
                                acc = acc + prod;
                            }
                            gp[IDX4(b, ci, ih, iw, C_in, Hp, Wp)] += acc;
                        }
                }
    for (int b = 0; b < B; ++b)
        for (int ci = 0; ci < C_in; ++ci)
            for (int h = 0; h < H; ++h)
                memcpy(dx + IDX4(b, ci, h, 0, C_in, H, W), gp + IDX4(b, ci, h + p_h, p_w, C_in, Hp, Wp),
                       sizeof(float) * W);
    free(gp);
}

/* _conv2d_backward_weight, nectarml/cpu/conv/conv2d.py:302-336.  Per (kh, kw):
 * einsum('bohw,bihw->oi', dY, strided patches of the padded input). */
void nml_oracle_conv2d_backward_weight(const float* dy, const float* x, float* dw, int B, int C_in, int H, int W,
                                       int C_out, int KH, int KW, int H_out, int W_out, int s_h, int s_w, int p_h,
                                       int p_w, int d_h, int d_w) {
    for (int co = 0; co < C_out; ++co)
        for (int ci = 0; ci < C_in; ++ci)
            for (int kh = 0; kh < KH; ++kh)
                for (int kw = 0; kw < KW; ++kw) {
                    float acc = 0.0f;
                    for (int b = 0; b < B; ++b)
                        for (int h = 0; h < H_out; ++h) {
                            int ih = h * s_h + kh * d_h - p_h;
                            if (ih < 0 || ih >= H) continue;
                            for (int wo = 0; wo < W_out; ++wo) {
                                int iw = wo * s_w + kw * d_w - p_w;
                                if (iw < 0 || iw >= W) continue;
                                float prod =
                                    dy[IDX4(b, co, h, wo, C_out, H_out, W_out)] * x[IDX4(b, ci, ih, iw, C_in, H, W)];
                                acc = acc + prod;
                            }
                        }
                    dw[IDX4(co, ci, kh, kw, C_in, KH, KW)] = acc;
                }
}

/* _conv_transpose2d_backward_input, nectarml/cpu/conv/conv2d.py:280-300: a plain _conv2d of the
 * output gradient with the same weight read as [C_out' = C_in][C_in' = C_out], no bias. */
void nml_oracle_conv_transpose2d_backward_input(const float* dy, const float* w, float* dx, int B, int C_in, int H,
                                                int W, int C_out, int KH, int KW, int H_out, int W_out, int s_h,
                                                int s_w, int p_h, int p_w, int d_h, int d_w) {
    nml_oracle_conv2d(dy, w, NULL, dx, B, C_out, H_out, W_out, C_in, KH, KW, H, W, s_h, s_w, p_h, p_w, d_h, d_w);
}

/* _conv_transpose2d_backward_weight, nectarml/cpu/conv/conv2d.py:338-378.  Per (kh, kw):
 * einsum('bihw,bohw->io', X, strided patches of the zero-padded dY). */
void nml_oracle_conv_transpose2d_backward_weight(const float* dy, const float* x, float* dw, int B, int C_in, int H,
                                                 int W, int C_out, int KH, int KW, int H_out, int W_out, int s_h,
                                                 int s_w, int p_h, int p_w, int d_h, int d_w) {
    for (int ci = 0; ci < C_in; ++ci)
        for (int co = 0; co < C_out; ++co)
            for (int kh = 0; kh < KH; ++kh)
                for (int kw = 0; kw < KW; ++kw) {
                    float acc = 0.0f;
                    for (int b = 0; b < B; ++b)
                        for (int h = 0; h < H; ++h) {
                            int oh = h * s_h + kh * d_h - p_h;
                            if (oh < 0 || oh >= H_out) continue;
                            for (int wi = 0; wi < W; ++wi) {
                                int ow = wi * s_w + kw * d_w - p_w;
                                if (ow < 0 || ow >= W_out) continue;
                                float prod =
                                    x[IDX4(b, ci, h, wi, C_in, H, W)] * dy[IDX4(b, co, oh, ow, C_out, H_out, W_out)];
                                acc = acc + prod;
                            }
                        }
                    dw[IDX4(ci, co, kh, kw, C_out, KH, KW)] = acc;
                }
}

/* `grad_output.sum(axis=(0, 2, 3))`, nectarml/cpu/conv/conv2d.py:64-67. */
void nml_oracle_bias_grad(const float* dy, float* db, int B, int C_out, int H_out, int W_out) {
    for (int co = 0; co < C_out; ++co) {
        double acc = 0.0; /* NumPy reduces pairwise; a double accumulator is at least as accurate */
        for (int b = 0; b < B; ++b)
            for (int i = 0; i < H_out * W_out; ++i) acc += dy[((size_t)b * C_out + co) * H_out * W_out + i];
        db[co] = (float)acc;
    }
}
