/*
 * CPU oracle for the dcgan-cuda convolution / Adam hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is a plain-C restatement of the
 * arithmetic of the reference's CPU backend (src/cpu/ops.hxx, src/cpu/kernels.cu).
 * It is the checker the CUDA path is compared against; nothing in the product
 * library links or calls it.
 *
 * Every function keeps the reference's floating-point evaluation order (which
 * scalar is accumulated in which order, where a double intermediate appears)
 * so that, compiled with -O2 -ffp-contract=off, it reproduces the reference
 * bit for bit (up to the sign of zero) on every configuration the reference's
 * CPU code handles.  It is pinned against the reference's own code compiled
 * from its sources (oracle/_ref, see ref_shim.cc) by tests/test_oracle.py and
 * against committed fixtures under tests/golden/.
 *
 * Layouts: activations NHWC, conv2d kernels HWIO [kh][kw][Cin][Cout],
 * conv2d_transpose kernels [kh][kw][Cout][Cin]; all fp32.
 */
#include <math.h>
#include <stddef.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define IDX4(n, h, w, c, H, W, C) ((((size_t)(n) * (H) + (h)) * (W) + (w)) * (C) + (c))

/* ---- xorshift, src/utils/xorshift.cu:11-40 ------------------------------- */
static uint64_t g_xs[4];

void orc_xorshift_seed(uint64_t x)
{
    g_xs[0] = 1000 * x;
    g_xs[1] = 2000 * x;
    g_xs[2] = 3000 * x;
    g_xs[3] = 4000 * x;
}

uint64_t orc_xorshift_next_u64(void)
{
    uint64_t t = g_xs[0] ^ (g_xs[0] << 11);
    g_xs[0] = g_xs[1];
    g_xs[1] = g_xs[2];
    g_xs[2] = g_xs[3];
    g_xs[3] = g_xs[3] ^ (g_xs[3] >> 19) ^ t ^ (t >> 8);
    return g_xs[3];
}

float orc_xorshift_next_f32(void)
{
    float x = (float)orc_xorshift_next_u64();
    float div = (float)0xFFFFFFFFFFFFFFFFull;
    return x / div;
}

void orc_xorshift_fill(float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = orc_xorshift_next_f32();
}

/* ---- conv2d forward, src/cpu/ops.hxx:188-267 ------------------------------
 * pad_h/pad_w are the TOTAL pads; top/left = total/2 (ops.hxx:204-205).
 * valid != 0: out = (in + pad - k)/stride + 1, else out = ceil(in/stride).
 * Accumulation order per output: channel, then kernel row, then kernel column
 * (ops.hxx:227-246); out-of-range taps are skipped. */
void orc_conv2d_out_size(int H, int W, int KH, int KW, int sh, int sw,
                         int pad_h, int pad_w, int valid, int* Ho, int* Wo)
{
    if (valid) {
        *Ho = (H + pad_h - KH) / sh + 1;
        *Wo = (W + pad_w - KW) / sw + 1;
    } else {
        *Ho = (int)ceilf((float)H / (float)sh);
        *Wo = (int)ceilf((float)W / (float)sw);
    }
}

void orc_conv2d(const float* x, const float* k, float* y,
                int N, int H, int W, int C, int KH, int KW, int O,
                int sh, int sw, int pad_h, int pad_w, int valid)
{
    int Ho, Wo;
    const int pt = pad_h / 2, pl = pad_w / 2;
    orc_conv2d_out_size(H, W, KH, KW, sh, sw, pad_h, pad_w, valid, &Ho, &Wo);
    for (int b = 0; b < N; ++b)
        for (int i = 0; i < Ho; ++i)
            for (int j = 0; j < Wo; ++j)
                for (int o = 0; o < O; ++o) {
                    float val = 0;
                    for (int q = 0; q < C; ++q)
                        for (int di = 0; di < KH; ++di)
                            for (int dj = 0; dj < KW; ++dj) {
                                int h = sh * i + di - pt;
                                int w = sw * j + dj - pl;
                                if (h >= 0 && w >= 0 && h < H && w < W)
                                    val += x[IDX4(b, h, w, q, H, W, C)] *
                                           k[IDX4(di, dj, q, o, KW, C, O)];
                            }
                    y[IDX4(b, i, j, o, Ho, Wo, O)] = val;
                }
}

/* ---- conv2d input gradient, src/cpu/ops.hxx:597-698 -----------------------
 * dy [N,Ho,Wo,O], k [KH,KW,C,O] -> dx [N,H,W,C].
 * The reference zero-inserts dy (stride-1 gaps), pads it with
 * pad = H - (s*(Ho-1)+1 - KH + 1), bottom = pad/2, top = pad - bottom
 * (ops.hxx:618-629), correlates each (channel, filter) pair with the
 * 180-degree rotated kernel and sums the per-filter results in filter order
 * (ops.hxx:650-679).  Terms that multiply an inserted zero do not change the
 * fp32 sum and are skipped here. */
void orc_conv2d_input_grad(const float* dy, const float* k, int stride,
                           int N, int Ho, int Wo, int O,
                           int KH, int KW, int C,
                           float* dx, int H, int W)
{
    const int sH = (Ho - 1) * (stride - 1) + Ho;
    const int sW = (Wo - 1) * (stride - 1) + Wo;
    const int pad_h = H - (sH - KH + 1);
    const int pad_w = W - (sW - KW + 1);
    const int pad_top = pad_h - pad_h / 2;
    const int pad_left = pad_w - pad_w / 2;

    for (int n = 0; n < N; ++n)
        for (int i = 0; i < H; ++i)
            for (int j = 0; j < W; ++j)
                for (int c = 0; c < C; ++c) {
                    float total = 0;
                    for (int o = 0; o < O; ++o) {
                        float val = 0;
                        for (int di = 0; di < KH; ++di) {
                            int ph = i + di - pad_top;
                            if (ph < 0 || ph % stride != 0) continue;
                            int a = ph / stride;
                            if (a >= Ho) continue;
                            for (int dj = 0; dj < KW; ++dj) {
                                int pw = j + dj - pad_left;
                                if (pw < 0 || pw % stride != 0) continue;
                                int b = pw / stride;
                                if (b >= Wo) continue;
                                val += dy[IDX4(n, a, b, o, Ho, Wo, O)] *
                                       k[IDX4(KH - 1 - di, KW - 1 - dj, c, o, KW, C, O)];
                            }
                        }
                        total = (o == 0) ? val : total + val;
                    }
                    dx[IDX4(n, i, j, c, H, W, C)] = total;
                }
}

/* ---- conv2d kernel gradient, src/cpu/ops.hxx:700-799 ----------------------
 * dy [N,Ho,Wo,O], x [N,H,W,C], total pads (pad_h,pad_w) -> dk [KH,KW,C,O]
 * with KH = H + pad_h - (s*(Ho-1)+1) + 1.  Per image the reference correlates
 * x with the zero-inserted dy (one fp32 accumulator per (kh,kw,c,o), scanned
 * row-major over dy), then adds the per-image results in image order
 * (ops.hxx:754-772). */
void orc_conv2d_kernel_grad_size(int H, int W, int Ho, int Wo, int stride,
                                 int pad_h, int pad_w, int* KH, int* KW)
{
    const int sH = (Ho - 1) * (stride - 1) + Ho;
    const int sW = (Wo - 1) * (stride - 1) + Wo;
    *KH = H + pad_h - sH + 1;
    *KW = W + pad_w - sW + 1;
}

void orc_conv2d_kernel_grad(const float* dy, const float* x, int stride,
                            int N, int Ho, int Wo, int O,
                            int H, int W, int C,
                            float* dk, int pad_h, int pad_w)
{
    int KH, KW;
    const int pt = pad_h / 2, pl = pad_w / 2;
    orc_conv2d_kernel_grad_size(H, W, Ho, Wo, stride, pad_h, pad_w, &KH, &KW);
    for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw)
            for (int c = 0; c < C; ++c)
                for (int o = 0; o < O; ++o) {
                    float total = 0;
                    for (int n = 0; n < N; ++n) {
                        float val = 0;
                        for (int a = 0; a < Ho; ++a) {
                            int h = kh + stride * a - pt;
                            if (h < 0 || h >= H) continue;
                            for (int b = 0; b < Wo; ++b) {
                                int w = kw + stride * b - pl;
                                if (w < 0 || w >= W) continue;
                                val += x[IDX4(n, h, w, c, H, W, C)] *
                                       dy[IDX4(n, a, b, o, Ho, Wo, O)];
                            }
                        }
                        total = (n == 0) ? val : total + val;
                    }
                    dk[IDX4(kh, kw, c, o, KW, C, O)] = total;
                }
}

/* ---- conv2d_transpose forward, src/cpu/ops.hxx:801-806 --------------------
 * x [N,Hx,Wx,Cx], k [KH,KW,Cy,Cx] -> y [N,Hy,Wy,Cy]: the input gradient of a
 * conv2d whose output is x. */
void orc_conv2d_transpose(const float* x, const float* k, int stride,
                          int N, int Hx, int Wx, int Cx,
                          int KH, int KW, int Cy,
                          float* y, int Hy, int Wy)
{
    orc_conv2d_input_grad(x, k, stride, N, Hx, Wx, Cx, KH, KW, Cy, y, Hy, Wy);
}

/* ---- conv2d_transpose input gradient --------------------------------------
 * dy [N,Hy,Wy,Cy], k [KH,KW,Cy,Cx] -> dx [N,Hx,Wx,Cx]: a strided conv2d of dy.
 * The reference's CPU code (src/cpu/ops.hxx:808-820) runs it with zero padding,
 * which is only the adjoint of conv2d_transpose when (Hx-1)*s + KH == Hy; its
 * GPU code (src/gpu/conv2d.cu:214-259) derives the pad from the input size.
 * This restatement uses the derived pad, which coincides with the CPU code
 * whenever that pad is zero. */
void orc_conv2d_transpose_input_grad(const float* dy, const float* k, int stride,
                                     int N, int Hy, int Wy, int Cy,
                                     int KH, int KW, int Cx,
                                     float* dx, int Hx, int Wx)
{
    const int pad_h = (Hx - 1) * stride + KH - Hy;
    const int pad_w = (Wx - 1) * stride + KW - Wy;
    orc_conv2d(dy, k, dx, N, Hy, Wy, Cy, KH, KW, Cx, stride, stride,
               pad_h, pad_w, 1);
}

/* ---- conv2d_transpose kernel gradient -------------------------------------
 * dy [N,Hy,Wy,Cy], x [N,Hx,Wx,Cx] -> dk [KH,KW,Cy,Cx].  Same structure as the
 * conv2d kernel gradient with the roles of the two activations swapped
 * (src/cpu/ops.hxx:822-902: per image, dy correlated with the zero-inserted x,
 * images summed in order).  Pad derived as in src/gpu/conv2d.cu:264-307; zero
 * pad reproduces the CPU code. */
void orc_conv2d_transpose_kernel_grad(const float* dy, const float* x, int stride,
                                      int N, int Hy, int Wy, int Cy,
                                      int Hx, int Wx, int Cx,
                                      float* dk, int KH, int KW)
{
    const int pad_h = (Hx - 1) * stride + KH - Hy;
    const int pad_w = (Wx - 1) * stride + KW - Wy;
    const int pt = pad_h / 2, pl = pad_w / 2;
    for (int kh = 0; kh < KH; ++kh)
        for (int kw = 0; kw < KW; ++kw)
            for (int cy = 0; cy < Cy; ++cy)
                for (int cx = 0; cx < Cx; ++cx) {
                    float total = 0;
                    for (int n = 0; n < N; ++n) {
                        float val = 0;
                        for (int a = 0; a < Hx; ++a) {
                            int h = kh + stride * a - pt;
                            if (h < 0 || h >= Hy) continue;
                            for (int b = 0; b < Wx; ++b) {
                                int w = kw + stride * b - pl;
                                if (w < 0 || w >= Wy) continue;
                                val += dy[IDX4(n, h, w, cy, Hy, Wy, Cy)] *
                                       x[IDX4(n, a, b, cx, Hx, Wx, Cx)];
                            }
                        }
                        total = (n == 0) ? val : total + val;
                    }
                    dk[IDX4(kh, kw, cy, cx, KW, Cy, Cx)] = total;
                }
}

/* ---- dense layers, src/cpu/ops.hxx:56-105,375-390 ------------------------- */
void orc_mm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < p; ++j) {
            float x = 0;
            for (size_t q = 0; q < n; ++q)
                x += a[i * n + q] * b[q * p + j];
            out[i * p + j] = x;
        }
}

/* out[m x p] = a^T b, a is [n x m], b is [n x p] */
void orc_tmm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < p; ++j) {
            float x = 0;
            for (size_t q = 0; q < n; ++q)
                x += a[q * m + i] * b[q * p + j];
            out[i * p + j] = x;
        }
}

/* out[m x p] = a b^T, a is [m x n], b is [p x n] */
void orc_mtm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < p; ++j) {
            float x = 0;
            for (size_t q = 0; q < n; ++q)
                x += a[i * n + q] * b[j * n + q];
            out[i * p + j] = x;
        }
}

void orc_mat_mul_add(const float* x, const float* w, const float* b, float* out,
                     size_t m, size_t n, size_t p)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < p; ++j) {
            float acc = 0;
            for (size_t q = 0; q < n; ++q)
                acc += x[i * n + q] * w[q * p + j];
            out[i * p + j] = acc + b[j];
        }
}

/* ---- bias add / bias grad, src/cpu/ops.hxx:107-117,405-416 ---------------- */
void orc_mvrow_add(const float* a, const float* b, float* out, size_t m, size_t n)
{
    for (size_t i = 0; i < m; ++i)
        for (size_t j = 0; j < n; ++j)
            out[i * n + j] = a[i * n + j] + b[j];
}

void orc_mat_sum_cols(const float* a, float* out, size_t m, size_t n)
{
    for (size_t i = 0; i < n; ++i) {
        float sum = 0;
        for (size_t j = 0; j < m; ++j)
            sum += a[j * n + i];
        out[i] = sum;
    }
}

void orc_mat_sum_rows(const float* a, float* out, size_t m, size_t n)
{
    for (size_t i = 0; i < m; ++i) {
        float sum = 0;
        for (size_t j = 0; j < n; ++j)
            sum += a[i * n + j];
        out[i] = sum;
    }
}

/* ---- activations, src/cpu/ops.hxx:13-17,312-359,423-466,926-931 -----------
 * sigmoid and tanh go through a double intermediate because the reference
 * writes them with double literals around a float exp. */
static float sigmoid_f(float x)
{
    return (float)(1.0 / (1.0 + (double)expf(-x)));
}

void orc_vect_sigmoid(const float* a, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = sigmoid_f(a[i]);
}

void orc_vect_relu(const float* a, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = a[i] < 0 ? 0 : a[i];
}

void orc_vect_relu_leaky(const float* a, float* out, size_t n, float alpha)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = a[i] < 0 ? alpha * a[i] : a[i];
}

void orc_vect_tanh(const float* a, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = (float)((2.0 / (1.0 + (double)expf(-2 * a[i]))) - 1.0);
}

void orc_relu_grad(const float* z, const float* dout, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = z[i] > 0 ? dout[i] : 0;
}

void orc_leaky_relu_grad(const float* z, const float* dout, float* out, float alpha, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = z[i] < 0 ? alpha * dout[i] : dout[i];
}

void orc_tanh_grad(const float* tanh_out, const float* dout, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = (float)((1 - pow((double)tanh_out[i], 2.0)) * (double)dout[i]);
}

void orc_sigmoid_grad(const float* sig_out, const float* dout, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = sig_out[i] * (1 - sig_out[i]) * dout[i];
}

/* ---- losses, src/cpu/ops.hxx:119-127,440-459 ------------------------------ */
float orc_sigmoid_cross_entropy(const float* y, const float* x, size_t n)
{
    float res = 0;
    for (size_t i = 0; i < n; ++i) {
        if (x[i] >= 0)
            res += x[i] - x[i] * y[i] + logf(1 + expf(-x[i]));
        else
            res += -x[i] * y[i] + logf(1 + expf(x[i]));
    }
    return res / n;
}

void orc_sigmoid_cross_entropy_grad(const float* y, const float* logits, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = (sigmoid_f(logits[i]) - y[i]) / n;
}

float orc_mse(const float* y, const float* y_hat, size_t m, size_t n)
{
    size_t len = m * n;
    float res = 0;
    for (size_t i = 0; i < len; ++i)
        res += (y[i] - y_hat[i]) * (y[i] - y_hat[i]);
    return res / len;
}

/* src/cpu/kernels.cu:112-115: out = (2/len) * (y_hat - y), coefficient in double
 * then narrowed to the float parameter of vect_sub_coeff. */
void orc_mse_grad(const float* y, const float* y_hat, float* out, size_t len)
{
    float coeff = (float)(2. / len);
    for (size_t i = 0; i < len; ++i)
        out[i] = coeff * (y_hat[i] - y[i]);
}

/* ---- elementwise, src/cpu/ops.hxx:432-438,933-939 ------------------------- */
void orc_vect_add(const float* a, const float* b, float* out, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = a[i] + b[i];
}

void orc_vect_update(const float* dv, float* out, float coeff, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] += coeff * dv[i];
}

/* ---- argmax accuracy, src/cpu/ops.hxx:38-46,468-476: first maximum wins ---- */
static size_t argmax_f(const float* v, size_t len)
{
    size_t res = 0;
    for (size_t i = 1; i < len; ++i)
        if (v[i] > v[res])
            res = i;
    return res;
}

float orc_argmax_acc(const float* y, const float* y_hat, size_t m, size_t n)
{
    size_t res = 0;
    for (size_t i = 0; i < m; ++i)
        res += argmax_f(y + i * n, n) == argmax_f(y_hat + i * n, n);
    return (float)res;
}

/* ---- Adam, src/cpu/ops.hxx:905-924 and src/cpu/kernels.cu:183-206 ---------- */
void orc_moment_update(const float* dv, float* out, float a, float b, size_t len)
{
    for (size_t i = 0; i < len; ++i)
        out[i] = a * out[i] + b * dv[i];
}

void orc_moment_update2(const float* dv, float* out, float a, float b, size_t len)
{
    for (size_t i = 0; i < len; ++i)
        out[i] = a * out[i] + b * dv[i] * dv[i];
}

/* Increments *t, returns the step size the reference derives from it. */
float orc_adam_lr_t(float* t, float lr, float beta1, float beta2)
{
    ++*t;
    return lr * sqrtf(1 - powf(beta2, *t)) / (1 - powf(beta1, *t));
}

void orc_adam_update(const float* m, const float* v, float* out, float lrt, float eps, size_t n)
{
    for (size_t i = 0; i < n; ++i)
        out[i] = out[i] - lrt * m[i] / (sqrtf(v[i]) + eps);
}
