// C-ABI wrapper around the reference's own CPU math (namespace cpu, header-only,
// src/cpu/ops.hh + ops.hxx).  TEST INFRASTRUCTURE ONLY.
//
// Compiled by oracle/build_oracle.py with the reference's source directory on
// the include path; the sources are used where they lie and are never copied
// into this repository.  The resulting library (oracle/_ref/libdcgan_ref_cpu.so)
// pins oracle/dcgan_oracle.c and can serve as the timed CPU baseline.
//
// Each wrapper forwards to exactly one reference entry point with the argument
// packing the reference's CPU dispatcher uses (src/cpu/kernels.cu:12-230).
#include <cstddef>
#include <cstring>

#include "cpu/ops.hh"

extern "C" {

// src/cpu/kernels.cu:12-18 -> cpu::conv2d (src/cpu/ops.hxx:257-267)
void ref_conv2d(const float* x, const float* k, float* y,
                const int* strides, int pad_h, int pad_w,
                const int* x_size, const int* k_size, int valid)
{
    cpu::conv2d(x, k, y, strides, pad_h, pad_w, x_size, k_size, valid);
}

// src/cpu/kernels.cu:32-35 -> cpu::conv2d_input_grad (ops.hxx:597-698)
void ref_conv2d_input_grad(const float* dy, const float* k, int stride,
                           const int* dy_size, const int* k_size,
                           float* out, const int* in_hw)
{
    cpu::conv2d_input_grad(dy, k, stride, dy_size, k_size, out, in_hw);
}

// src/cpu/kernels.cu:37-40 -> cpu::conv2d_kernel_grad (ops.hxx:700-799)
void ref_conv2d_kernel_grad(const float* dy, const float* x, int stride,
                            const int* dy_size, const int* x_size,
                            float* out, const int* pad_hw)
{
    cpu::conv2d_kernel_grad(dy, x, stride, dy_size, x_size, out, pad_hw);
}

// src/cpu/kernels.cu:42-45 -> cpu::conv2d_transpose (ops.hxx:801-806)
void ref_conv2d_transpose(const float* x, const float* k, const int* out_size,
                          int stride, float* out, const int* x_size,
                          const int* k_size)
{
    cpu::conv2d_transpose(x, k, out_size, stride, out, x_size, k_size);
}

// src/cpu/kernels.cu:47-50 -> cpu::conv2d_transpose_input_grad (ops.hxx:808-820)
void ref_conv2d_transpose_input_grad(const float* dy, const float* k, int stride,
                                     const int* dy_size, const int* k_size,
                                     float* out, const int* in_hw)
{
    cpu::conv2d_transpose_input_grad(dy, k, stride, dy_size, k_size, out, in_hw);
}

// src/cpu/kernels.cu:52-55 -> cpu::conv2d_transpose_kernel_grad (ops.hxx:822-902)
void ref_conv2d_transpose_kernel_grad(const float* dy, const float* x, int stride,
                                      const int* dy_size, const int* x_size,
                                      float* out)
{
    cpu::conv2d_transpose_kernel_grad(dy, x, stride, dy_size, x_size, out);
}

void ref_mm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{ cpu::mm_mul(a, b, out, m, n, p); }
void ref_tmm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{ cpu::tmm_mul(a, b, out, m, n, p); }
void ref_mtm_mul(const float* a, const float* b, float* out, size_t m, size_t n, size_t p)
{ cpu::mtm_mul(a, b, out, m, n, p); }
void ref_mat_mul_add(const float* x, const float* w, const float* b, float* out,
                     size_t m, size_t n, size_t p)
{ cpu::mat_mul_add(x, w, b, out, m, n, p); }
void ref_mvrow_add(const float* a, const float* b, float* out, size_t m, size_t n)
{ cpu::mvrow_add(a, b, out, m, n); }
void ref_mat_sum_cols(const float* a, float* out, size_t m, size_t n)
{ cpu::mat_sum_cols(a, out, m, n); }
void ref_mat_sum_rows(const float* a, float* out, size_t m, size_t n)
{ cpu::mat_sum_rows(a, out, m, n); }

void ref_vect_sigmoid(const float* a, float* out, size_t n) { cpu::vect_sigmoid(a, out, n); }
void ref_vect_relu(const float* a, float* out, size_t n) { cpu::vect_relu(a, out, n); }
void ref_vect_relu_leaky(const float* a, float* out, size_t n, float alpha)
{ cpu::vect_relu_leaky(a, out, n, alpha); }
void ref_vect_tanh(const float* a, float* out, size_t n) { cpu::vect_tanh(a, out, n); }
void ref_relu_grad(const float* z, const float* dout, float* out, size_t n)
{ cpu::relu_grad(z, dout, out, n); }
void ref_leaky_relu_grad(const float* z, const float* dout, float* out, float alpha, size_t n)
{ cpu::leaky_relu_grad(z, dout, out, alpha, n); }
void ref_tanh_grad(const float* t, const float* dout, float* out, size_t n)
{ cpu::tanh_grad(t, dout, out, n); }
void ref_sigmoid_grad(const float* s, const float* dout, float* out, size_t n)
{ cpu::sigmoid_grad(s, dout, out, n); }

float ref_sigmoid_cross_entropy(const float* y, const float* x, size_t n)
{ return cpu::sigmoid_cross_entropy(y, x, n); }
void ref_sigmoid_cross_entropy_grad(const float* y, const float* x, float* out, size_t n)
{ cpu::sigmoid_cross_entropy_grad(y, x, out, n); }
float ref_mse(const float* y, const float* y_hat, size_t m, size_t n)
{ return cpu::mse(y, y_hat, m, n); }
// src/cpu/kernels.cu:112-115
void ref_mse_grad(const float* y, const float* y_hat, float* out, size_t len)
{ cpu::vect_sub_coeff(y_hat, y, 2. / len, out, len); }

void ref_vect_add(const float* a, const float* b, float* out, size_t n)
{ cpu::vect_add(a, b, out, n); }
void ref_vect_update(const float* dv, float* out, float coeff, size_t n)
{ cpu::vect_update(dv, out, coeff, n); }
float ref_argmax_acc(const float* y, const float* y_hat, size_t m, size_t n)
{ return (float)cpu::argmax_acc(y, y_hat, m, n); }

void ref_moment_update(const float* dv, float* out, float a, float b, size_t n)
{ cpu::moment_update(dv, out, a, b, n); }
void ref_moment_update2(const float* dv, float* out, float a, float b, size_t n)
{ cpu::moment_update2(dv, out, a, b, n); }
// src/cpu/kernels.cu:193-206
float ref_adam_lr_t(float* t, float lr, float beta1, float beta2)
{
    ++*t;
    return lr * std::sqrt(1 - std::pow(beta2, *t)) / (1 - std::pow(beta1, *t));
}
void ref_adam_update(const float* m, const float* v, float* out, float lrt, float eps, size_t n)
{ cpu::adam_update(m, v, out, lrt, eps, n); }

}  // extern "C"

// src/utils/xorshift.cu:11-40 (compiled from the reference beside this file)
#include "utils/xorshift.hh"
extern "C" {
void ref_xorshift_seed(unsigned long long x) { xorshift::seed(x); }
unsigned long long ref_xorshift_next_u64() { return xorshift::next_u64(); }
float ref_xorshift_next_f32() { return xorshift::next_f32(); }
void ref_xorshift_fill(float* out, size_t n) { xorshift::fill(out, out + n); }
}
