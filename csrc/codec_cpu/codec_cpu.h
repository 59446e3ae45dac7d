// CPU codecs: the byte-exact specification of every payload in executable form.
//
// These are plain C++17 loops over raw pointers (no Thrust, no torch).  They
// serve three purposes: (1) the oracle the sm_100a kernels are byte-compared
// against in tests, (2) the backend of the task runtime when it is handed CPU
// tensors, (3) the timed CPU baseline of the codec round-trip benchmark.
// Behavioural parity targets are the reference's host-policy instantiations of
// ZQ_CPP_LIB/gradient_compression_body/{tbq,terngrad,gd,dgc,ecq}_body.h.
#pragma once
#include <stdint.h>

namespace hipress {
namespace cpu {

// Worker threads the TBQ and TernGrad codecs may split a tensor over (default 1: the plain
// loops).  Every payload byte depends on its own 4 (or 8 / bitwidth) elements only -- the
// stochastic rounding is seeded per byte -- so the split changes no bit of payload, residual or
// decode.  The min/max pass of the TernGrad compressor stays sequential (its first-minimum /
// last-maximum rule is defined by element order).  Tensors below 2^16 elements per thread are
// not split.  The reference's host path is single-threaded.
void set_threads(int threads);
int get_threads();

// ---- TBQ (ref tbq_body.h:90-158 compress, :160-200 decompress)
// out must hold ceil(n/4) bytes.  residual is updated in place; grad is not.
void tbq_compress(const float* grad, float* residual, int64_t n, float threshold, uint8_t* out);
// Decodes exactly n elements; add != 0 accumulates into out.
void tbq_decompress(const uint8_t* in, int64_t n, float threshold, float* out, int add);

// ---- TernGrad-style min-max k-bit quantiser (ref terngrad_body.h:162-307, :309-409)
// out_size must equal 10 + ceil(n/dpb).  `residual` may be null; when given,
// the quantised tensor is grad + residual and residual receives the
// quantisation error (error feedback).  Returns 0, or -1 for a bad bitwidth /
// buffer size.
int terngrad_compress(const float* grad, int64_t n, int bitwidth, int enable_random, uint64_t seed,
                      uint8_t* out, int64_t out_size, float* residual);
// Decodes ((in_size-10)*dpb - tail) elements taken from the header; returns
// that count, or -1 on a malformed header / too small `out_capacity`.
int64_t terngrad_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t out_capacity,
                            int add);

// ---- Sampled-threshold top-k sparsifier (GradDrop: ref gd_body.h:102-232;
// DGC: ref dgc_body.h:154-229; decode ref gd_body.h:283-353)
// accumulate != 0 (GradDrop): R += grad first, then select from R.
// accumulate == 0 (DGC): `grad` is ignored and R is the tensor selected from.
// Selected entries of R are zeroed.  keep_fraction = 1 - drop_ratio.
// Deterministic content rule: threshold = the sample of rank
// (int)(sample_cnt*keep_fraction) in descending |.| order; keep |R[i]| > threshold
// in ascending index order; when more than ceil(n*keep_fraction) qualify, keep
// the largest magnitudes with ties broken toward the lower index, still emitted
// in ascending index order.  Returns payload bytes written, or -1 if
// out_capacity is too small for the worst case 4 + 8*ceil(n*keep_fraction).
int64_t sparse_compress(const float* grad, float* R, int64_t n, double sample_rate,
                        double keep_fraction, uint64_t seed, int accumulate, uint8_t* out,
                        int64_t out_capacity);
// add != 0: out[idx] += val; else zero-fill n elements then scatter.
// Returns k, or -1 if the header exceeds in_size or an index is out of range.
int64_t sparse_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t n, int add);

// ---- ECQ (layout per ref ecq_body.h:266-276; corrected semantics: the sign of
// G + alpha*H is kept, every data byte is produced, header written after max is known)
int ecq_compress(const float* grad, float* history, int64_t n, float alpha, float beta,
                 int bitwidth, uint64_t seed, uint8_t* out, int64_t out_size);
int64_t ecq_decompress(const uint8_t* in, int64_t in_size, float* out, int64_t out_capacity,
                       int add);

// ---- PowerSGD, intended maths of ref powersgd_body.h:10-78 (the shipped code
// discards its results).  Row-major fp32; M is n x m, P is n x r, Q is m x r.
// encode1: M[:N] = grad + residual; P = M Q
void powersgd_encode1(const float* grad, const float* residual, int64_t N, float* M, int64_t n,
                      int64_t m, const float* Q, int64_t r, float* P);
// encode2: P = orthonormalise(P) (modified Gram-Schmidt, column by column); Q = M^T P
void powersgd_encode2(float* P, const float* M, int64_t n, int64_t m, int64_t r, float* Q);
// decode: M = P Q^T; residual = grad - M[:N]; grad = M[:N]
void powersgd_decode(const float* P, const float* Q, int64_t n, int64_t m, int64_t r, float* M,
                     float* residual, float* grad, int64_t N);
// Column-wise modified Gram-Schmidt on an n x r row-major matrix, in place.
// Column norms below eps are replaced by eps before dividing.
void gram_schmidt(float* P, int64_t n, int64_t r, float eps);

}  // namespace cpu
}  // namespace hipress
