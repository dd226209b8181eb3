// leopard_b200 — glue kernels of models whose residual stream is kept in 32-bit floats.
//
//   lp_embed_rows_f32   x[r, :] = table[ids[r], :] * scale  (bf16 table -> fp32 rows)
//   lp_rmsnorm_f32      y = x / sqrt(mean(x^2) + eps) * g over fp32 rows, eps inside the root; g is one number (gain_scalar), a vector
//                       (gain_vec) or both.  The result is written as fp32 or bf16 (the operand of the next matrix product), or — with
//                       `accum` — added to another fp32 matrix: the sandwich-norm residual update x <- x + norm(sublayer(x)) in one pass.
//   lp_glu_f32          elementwise epilogues for matrix products that ran elsewhere: xIELU, squared relu, silu(gate) * up.
//   lp_axpy_f32         y <- y + alpha x, the residual update after such a product.
//   lp_add_positions_f32  x[r, 2i] += sin(p f_i), x[r, 2i + 1] += cos(p f_i) with p the row's position: absolute sinusoidal positions
//                       added to the stream (fp32 angles with the product's rounding error carried along, accurate sincosf).
//   lp_add_row_f32      x[r, :] += v for every row (a learned vector that marks a pass of a looped stack).
//   lp_token_shift_f32  y_t = h_t + (h_(t-1) - h_t) * mu per channel, with h the rows as they came in; the row before a request's
//                       first row of this step comes from the request's slot (zeros at position 0), and the slot then takes the
//                       request's last row.
//   lp_dyt_f32          Dynamic Tanh: tanh(alpha x) * gain + shift per element, no statistics; one pass can serve the two sublayers of a
//                       parallel layer (two parameter sets, two outputs).
//   lp_rmsnorm_gated_f32  the RMS norm with a vector gain, multiplied by sigmoid(gate) per element (norm over a mixer's concatenated
//                       heads and its output gate in one pass).
//   lp_gated_axpy_f32   x <- x + mult (y + y_bias) sigmoid(g + g_bias): a residual branch behind a learned gate.
//   lp_depth_average_f32  out = sum_j coef[j] X_j over the results of all layers so far (and a copy of it for the next layer's branches).
//
// One warp per row, statistics and normalisation in fp32; the row is read twice (the second read hits L1 / L2).
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

__global__ void embed_rows_f32_kernel(const int* __restrict__ ids, int R, const bf16* __restrict__ table, long long ldt, int vocab,
                                      float scale, float* __restrict__ out, long long ldo, int D) {
  const int r = blockIdx.x;
  if (r >= R) return;
  int id = ids[r];
  if (id < 0 || id >= vocab) id = 0;   // the host validates ids; this only keeps a bad one inside the table
  const bf16* src = table + (long long)id * ldt;
  float* dst = out + (long long)r * ldo;
  for (int c = threadIdx.x; c < D; c += blockDim.x) dst[c] = __bfloat162float(src[c]) * scale;
}

constexpr int NORM32_WARPS = 8;
__global__ void __launch_bounds__(NORM32_WARPS * 32)
rmsnorm_f32_kernel(const float* __restrict__ x, long long ldx, int M, int D, float gain_scalar, const float* __restrict__ gain_vec,
                   float eps, float* __restrict__ out_f32, bf16* __restrict__ out_bf16, long long ldo, float* __restrict__ accum,
                   long long lda) {
  const int row = blockIdx.x * NORM32_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float* xr = x + (long long)row * ldx;
  float ss = 0.f;
  for (int c = lane; c < D; c += 32) {
    const float v = xr[c];
    ss = fmaf(v, v, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  for (int c = lane; c < D; c += 32) {
    float v = xr[c] * r * gain_scalar;
    if (gain_vec != nullptr) v *= gain_vec[c];
    if (accum != nullptr) accum[(long long)row * lda + c] += v;
    else if (out_f32 != nullptr) out_f32[(long long)row * ldo + c] = v;
    else out_bf16[(long long)row * ldo + c] = __float2bfloat16(v);
  }
}

template <typename T> __device__ __forceinline__ float ld32(const T* p);
template <> __device__ __forceinline__ float ld32<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float ld32<bf16>(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void st32(float* p, float v) { *p = v; }
__device__ __forceinline__ void st32(bf16* p, float v) { *p = __float2bfloat16(v); }

// mode LP_EPI_XIELU: out[m, n] = xielu(in[m, n]); LP_EPI_SILU_GATE: out[m, n] = silu(in[m, n]) * in[m, n + N]; LP_EPI_CLAMP_GLU: the
// clamped gated unit of lp_linear on (in[m, n], in[m, n + N]) with limit a and slope b.  row_scale multiplies what is read.
template <typename IT, typename OT>
__global__ void glu_kernel(const IT* __restrict__ in, long long ldi, OT* __restrict__ out, long long ldo, int M, int N, int mode, float a,
                           float b, const float* __restrict__ row_scale) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  const float rs = row_scale != nullptr ? row_scale[m] : 1.0f;
  const float z = ld32<IT>(in + (long long)m * ldi + n) * rs;
  float v;
  if (mode == LP_EPI_SILU_GATE) v = z / (1.0f + expf(-z)) * (ld32<IT>(in + (long long)m * ldi + n + N) * rs);
  else if (mode == LP_EPI_CLAMP_GLU) {
    const float g = fminf(z, a), u = fminf(fmaxf(ld32<IT>(in + (long long)m * ldi + n + N) * rs, -a), a);
    v = g / (1.0f + expf(-b * g)) * (u + 1.0f);
  }
  else if (mode == LP_EPI_RELU2) v = fmaxf(z, 0.f) * fmaxf(z, 0.f);
  else v = z > 0.f ? a * z * z + 0.5f * z : b * (expm1f(z) - z) + 0.5f * z;
  st32(out + (long long)m * ldo + n, v);
}

// The three elementwise kernels below work on groups of V consecutive columns per thread: V = 4 (16-byte fp32 accesses, 8-byte bf16
// stores) when the width and every row stride and base allow it, else V = 1.
template <int V> struct f32vec;
template <> struct f32vec<1> { float v[1]; };
template <> struct alignas(16) f32vec<4> { float v[4]; };
template <int V> __device__ __forceinline__ f32vec<V> ldv(const float* p) { return *reinterpret_cast<const f32vec<V>*>(p); }
template <int V> __device__ __forceinline__ void stv(float* p, const f32vec<V>& x) { *reinterpret_cast<f32vec<V>*>(p) = x; }
template <int V> __device__ __forceinline__ void stv(bf16* p, const f32vec<V>& x) {
  if constexpr (V == 4) {
    const __nv_bfloat162 lo = __floats2bfloat162_rn(x.v[0], x.v[1]), hi = __floats2bfloat162_rn(x.v[2], x.v[3]);
    uint2 u;
    u.x = *reinterpret_cast<const unsigned*>(&lo);
    u.y = *reinterpret_cast<const unsigned*>(&hi);
    *reinterpret_cast<uint2*>(p) = u;
  } else {
    *p = __float2bfloat16(x.v[0]);
  }
}

// a warp per row; the lanes take groups of V consecutive columns (V = 4: 16-byte reads of the row and of its gate)
template <typename OT, int V>
__global__ void __launch_bounds__(NORM32_WARPS * 32)
rmsnorm_gated_f32_kernel(const float* __restrict__ x, long long ldx, int M, int D, const float* __restrict__ gain, float eps,
                         const float* __restrict__ gate, long long ldg, OT* __restrict__ out, long long ldo) {
  const int row = blockIdx.x * NORM32_WARPS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (row >= M) return;
  const float* xr = x + (long long)row * ldx;
  float ss = 0.f;
  for (int c = lane * V; c < D; c += 32 * V) {
    const f32vec<V> v = ldv<V>(xr + c);
#pragma unroll
    for (int k = 0; k < V; ++k) ss = fmaf(v.v[k], v.v[k], ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float r = 1.0f / sqrtf(ss / (float)D + eps);
  for (int c = lane * V; c < D; c += 32 * V) {
    f32vec<V> v = ldv<V>(xr + c);
    const f32vec<V> g = ldv<V>(gate + (long long)row * ldg + c);
#pragma unroll
    for (int k = 0; k < V; ++k) {
      v.v[k] *= r;
      if (gain != nullptr) v.v[k] *= gain[c + k];
      v.v[k] /= 1.0f + expf(-g.v[k]);
    }
    stv<V>(out + (long long)row * ldo + c, v);
  }
}

// tanh for an output that is rounded to bf16 (8 bits of mantissa): 1 - 2 / (e^(2|x|) + 1) on the fast exponential and division
// (absolute error of a few 1e-7, far below the rounding that follows); the fp32 output keeps the accurate tanhf
template <typename OT> __device__ __forceinline__ float dyt_tanh(float x);
template <> __device__ __forceinline__ float dyt_tanh<float>(float x) { return tanhf(x); }
template <> __device__ __forceinline__ float dyt_tanh<bf16>(float x) {
  const float a = fminf(fabsf(x), 15.f);      // tanh(15) rounds to 1 in fp32; the bound keeps the exponential finite
  const float t = 1.0f - __fdividef(2.0f, __expf(2.0f * a) + 1.0f);
  return copysignf(t, x);
}

template <typename OT, int V>
__global__ void dyt_f32_kernel(const float* __restrict__ x, long long ldx, int M, int D, float alpha, const float* __restrict__ gain,
                               const float* __restrict__ shift, OT* __restrict__ out, long long ldo, float alpha2,
                               const float* __restrict__ gain2, const float* __restrict__ shift2, OT* __restrict__ out2, long long ldo2) {
  const int DV = D / V;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * DV) return;
  const int m = (int)(i / DV), c = (int)(i % DV) * V;
  const f32vec<V> v = ldv<V>(x + (long long)m * ldx + c);
  f32vec<V> y;
  {
    const f32vec<V> g = ldv<V>(gain + c);
#pragma unroll
    for (int k = 0; k < V; ++k) y.v[k] = fmaf(dyt_tanh<OT>(alpha * v.v[k]), g.v[k], shift != nullptr ? shift[c + k] : 0.f);
    stv<V>(out + (long long)m * ldo + c, y);
  }
  if (out2 != nullptr) {
    const f32vec<V> g = ldv<V>(gain2 + c);
#pragma unroll
    for (int k = 0; k < V; ++k) y.v[k] = fmaf(dyt_tanh<OT>(alpha2 * v.v[k]), g.v[k], shift2 != nullptr ? shift2[c + k] : 0.f);
    stv<V>(out2 + (long long)m * ldo2 + c, y);
  }
}

template <int V>
__global__ void gated_axpy_f32_kernel(float* __restrict__ x, long long ldx, const float* __restrict__ y, long long ldy,
                                      const float* __restrict__ y_bias, const float* __restrict__ g, long long ldg,
                                      const float* __restrict__ g_bias, float mult, int M, int N) {
  const int NV = N / V;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * NV) return;
  const int m = (int)(i / NV), n = (int)(i % NV) * V;
  f32vec<V> acc = ldv<V>(x + (long long)m * ldx + n);
  const f32vec<V> yv = ldv<V>(y + (long long)m * ldy + n);
  f32vec<V> gv;
  if (g != nullptr) gv = ldv<V>(g + (long long)m * ldg + n);
#pragma unroll
  for (int k = 0; k < V; ++k) {
    float v = yv.v[k] + (y_bias != nullptr ? y_bias[n + k] : 0.f);
    if (g != nullptr) v /= 1.0f + expf(-(gv.v[k] + (g_bias != nullptr ? g_bias[n + k] : 0.f)));
    acc.v[k] = fmaf(mult, v, acc.v[k]);
  }
  stv<V>(x + (long long)m * ldx + n, acc);
}

template <int V>
__global__ void depth_average_f32_kernel(const float* __restrict__ hist, long long layer_stride, long long ldh,
                                         const float* __restrict__ coef, int n, float* __restrict__ out, long long ldo,
                                         float* __restrict__ copy, long long ldc, int M, int N) {
  const int NV = N / V;
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * NV) return;
  const int m = (int)(i / NV), c = (int)(i % NV) * V;
  const float* src = hist + (long long)m * ldh + c;
  f32vec<V> acc;
#pragma unroll
  for (int k = 0; k < V; ++k) acc.v[k] = 0.f;
  for (int j = 0; j < n; ++j) {
    const f32vec<V> h = ldv<V>(src + (long long)j * layer_stride);
    const float cj = coef[j];
#pragma unroll
    for (int k = 0; k < V; ++k) acc.v[k] = fmaf(cj, h.v[k], acc.v[k]);
  }
  stv<V>(out + (long long)m * ldo + c, acc);
  if (copy != nullptr) stv<V>(copy + (long long)m * ldc + c, acc);
}

// 16-byte accesses need every base on a 16-byte boundary and every row stride a multiple of four floats
static bool vec4_ok(int N, std::initializer_list<const void*> bases, std::initializer_list<long long> strides) {
  if (N % 4) return false;
  for (const void* b : bases)
    if (b != nullptr && (reinterpret_cast<uintptr_t>(b) & 15)) return false;
  for (long long s : strides)
    if (s % 4) return false;
  return true;
}

__global__ void axpy_f32_kernel(float* __restrict__ y, long long ldy, const float* __restrict__ x, long long ldx, float alpha, int M, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  y[(long long)m * ldy + n] = fmaf(alpha, x[(long long)m * ldx + n], y[(long long)m * ldy + n]);
}

// pair i of a row: (sin, cos) of position * frequency i; an odd width leaves the last sine without its cosine.  The frequency comes as
// two floats hi + lo (a float64 value split once on the host), and the product's rounding error is recovered with one fma, so the
// angle is a = fl(p hi) plus a small rest e known to about 2^-48 of a: sin(a + e) = sin a + e cos a, cos(a + e) = cos a - e sin a.
__global__ void add_positions_f32_kernel(float* __restrict__ x, long long ldx, int R, int D, const int* __restrict__ row_pos,
                                         const float* __restrict__ freq, int n_freq) {
  const int r = blockIdx.x;
  if (r >= R) return;
  const float p = (float)row_pos[r];
  float* xr = x + (long long)r * ldx;
  for (int i = threadIdx.x; 2 * i < D; i += blockDim.x) {
    const float hi = freq[i], lo = freq[n_freq + i];
    const float a = p * hi;
    const float e = fmaf(p, hi, -a) + p * lo;
    float s, c;
    sincosf(a, &s, &c);
    xr[2 * i] += fmaf(e, c, s);
    if (2 * i + 1 < D) xr[2 * i + 1] += fmaf(-e, s, c);
  }
}

__global__ void add_row_f32_kernel(float* __restrict__ x, long long ldx, const float* __restrict__ v, int M, int N) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)M * N) return;
  const int m = (int)(i / N), n = (int)(i % N);
  x[(long long)m * ldx + n] += v[n];
}

// One thread per (row, channel).  Only the thread of a request's FIRST row touches the request's slot: it reads the carried row
// and then stores the request's last row of this step there, so no other thread of the launch reads what it writes.
template <typename OT>
__global__ void token_shift_kernel(const float* __restrict__ h, long long ldh, const float* __restrict__ mu, int R, int D,
                                   const int* __restrict__ row_seq, const int* __restrict__ row_pos, const int* __restrict__ seq_row0,
                                   const int* __restrict__ seq_slot, float* __restrict__ state, long long slot_stride,
                                   OT* __restrict__ out, long long ldo) {
  const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= (long long)R * D) return;
  const int r = (int)(i / D), c = (int)(i % D);
  const int s = row_seq[r];
  const float cur = h[(long long)r * ldh + c];
  float prev;
  if (r == seq_row0[s]) {
    float* slot = state + (long long)seq_slot[s] * slot_stride;
    prev = row_pos[r] > 0 ? slot[c] : 0.f;
    slot[c] = h[(long long)(seq_row0[s + 1] - 1) * ldh + c];
  } else {
    prev = h[(long long)(r - 1) * ldh + c];
  }
  st32(out + (long long)r * ldo + c, fmaf(prev - cur, mu[c], cur));
}

}  // namespace lp

using namespace lp;

extern "C" int lp_add_positions_f32(float* x, long long ldx, int R, int D, const int* row_pos, const float* freq, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && row_pos != nullptr && freq != nullptr && R >= 0 && D > 0, "lp_add_positions_f32: bad arguments");
  if (R == 0) return 0;
  add_positions_f32_kernel<<<R, 128, 0, stream>>>(x, ldx, R, D, row_pos, freq, (D + 1) / 2);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_add_row_f32(float* x, long long ldx, const float* v, int M, int N, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && v != nullptr && M >= 0 && N > 0, "lp_add_row_f32: bad arguments");
  if (M == 0) return 0;
  add_row_f32_kernel<<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, stream>>>(x, ldx, v, M, N);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_token_shift_f32(const float* h, long long ldh, const float* mu, int R, int D, const int* row_seq, const int* row_pos,
                                  const int* seq_row0, const int* seq_slot, float* state, long long slot_stride, void* out,
                                  long long ldo, int out_fp32, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(h != nullptr && mu != nullptr && out != nullptr && state != nullptr && row_seq != nullptr && row_pos != nullptr &&
                 seq_row0 != nullptr && seq_slot != nullptr && R >= 0 && D > 0 && slot_stride >= D,
             "lp_token_shift_f32: bad arguments");
  LP_REQUIRE(h != out, "lp_token_shift_f32: a row reads its neighbour as it came in, so it cannot run in place");
  if (R == 0) return 0;
  const unsigned grid = (unsigned)(((long long)R * D + 255) / 256);
  if (out_fp32)
    token_shift_kernel<float><<<grid, 256, 0, stream>>>(h, ldh, mu, R, D, row_seq, row_pos, seq_row0, seq_slot, state, slot_stride,
                                                        reinterpret_cast<float*>(out), ldo);
  else
    token_shift_kernel<bf16><<<grid, 256, 0, stream>>>(h, ldh, mu, R, D, row_seq, row_pos, seq_row0, seq_slot, state, slot_stride,
                                                       reinterpret_cast<bf16*>(out), ldo);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_embed_rows_f32(const int* ids, int R, const void* table, long long ldt, int vocab, float scale, float* out, long long ldo,
                                 int D, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(ids != nullptr && table != nullptr && out != nullptr && R >= 0 && D > 0 && vocab > 0, "lp_embed_rows_f32: bad arguments");
  if (R == 0) return 0;
  embed_rows_f32_kernel<<<R, 128, 0, stream>>>(ids, R, reinterpret_cast<const bf16*>(table), ldt, vocab, scale, out, ldo, D);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_rmsnorm_f32(const float* x, long long ldx, int M, int D, float gain_scalar, const float* gain_vec, float eps, void* out,
                              long long ldo, int out_fp32, float* accum, long long ld_accum, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && M >= 0 && D > 0, "lp_rmsnorm_f32: bad arguments");
  LP_REQUIRE((out != nullptr) != (accum != nullptr), "lp_rmsnorm_f32: give either `out` or `accum`");
  if (M == 0) return 0;
  rmsnorm_f32_kernel<<<(M + NORM32_WARPS - 1) / NORM32_WARPS, NORM32_WARPS * 32, 0, stream>>>(
      x, ldx, M, D, gain_scalar, gain_vec, eps, (out != nullptr && out_fp32) ? reinterpret_cast<float*>(out) : nullptr,
      (out != nullptr && !out_fp32) ? reinterpret_cast<bf16*>(out) : nullptr, ldo, accum, ld_accum);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_glu_f32(const void* in, long long ldi, int in_fp32, void* out, long long ldo, int out_fp32, int M, int N, int mode,
                          float a, float b, void* stream_) {
  return lp_glu_scaled_f32(in, ldi, in_fp32, out, ldo, out_fp32, M, N, mode, a, b, nullptr, stream_);
}

extern "C" int lp_glu_scaled_f32(const void* in, long long ldi, int in_fp32, void* out, long long ldo, int out_fp32, int M, int N, int mode,
                                 float a, float b, const float* row_scale, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(in != nullptr && out != nullptr && M >= 0 && N > 0, "lp_glu_f32: bad arguments");
  LP_REQUIRE(mode == LP_EPI_XIELU || mode == LP_EPI_SILU_GATE || mode == LP_EPI_RELU2 || mode == LP_EPI_CLAMP_GLU,
             "lp_glu_f32: mode %d is not an activation", mode);
  if (M == 0) return 0;
  const unsigned grid = (unsigned)(((long long)M * N + 255) / 256);
  if (in_fp32 && out_fp32)
    glu_kernel<float, float><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(in), ldi, reinterpret_cast<float*>(out), ldo, M, N, mode, a, b, row_scale);
  else if (in_fp32)
    glu_kernel<float, bf16><<<grid, 256, 0, stream>>>(reinterpret_cast<const float*>(in), ldi, reinterpret_cast<bf16*>(out), ldo, M, N, mode, a, b, row_scale);
  else if (out_fp32)
    glu_kernel<bf16, float><<<grid, 256, 0, stream>>>(reinterpret_cast<const bf16*>(in), ldi, reinterpret_cast<float*>(out), ldo, M, N, mode, a, b, row_scale);
  else
    glu_kernel<bf16, bf16><<<grid, 256, 0, stream>>>(reinterpret_cast<const bf16*>(in), ldi, reinterpret_cast<bf16*>(out), ldo, M, N, mode, a, b, row_scale);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_dyt_f32(const float* x, long long ldx, int M, int D, float alpha, const float* gain, const float* shift, void* out,
                          long long ldo, float alpha2, const float* gain2, const float* shift2, void* out2, long long ldo2, int out_fp32,
                          void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && gain != nullptr && out != nullptr && M >= 0 && D > 0, "lp_dyt_f32: bad arguments");
  LP_REQUIRE(out2 == nullptr || gain2 != nullptr, "lp_dyt_f32: a second output without its gain");
  if (M == 0) return 0;
  // bf16 rows of four are 8 bytes: their bases need 8-byte alignment, which the 16-byte test covers
  const bool v4 = vec4_ok(D, {x, gain, gain2, out, out2}, {ldx, ldo, out2 != nullptr ? ldo2 : 0});
  const unsigned grid = (unsigned)(((long long)M * (v4 ? D / 4 : D) + 255) / 256);
  if (out_fp32 && v4)
    dyt_f32_kernel<float, 4><<<grid, 256, 0, stream>>>(x, ldx, M, D, alpha, gain, shift, reinterpret_cast<float*>(out), ldo, alpha2, gain2,
                                                       shift2, reinterpret_cast<float*>(out2), ldo2);
  else if (out_fp32)
    dyt_f32_kernel<float, 1><<<grid, 256, 0, stream>>>(x, ldx, M, D, alpha, gain, shift, reinterpret_cast<float*>(out), ldo, alpha2, gain2,
                                                       shift2, reinterpret_cast<float*>(out2), ldo2);
  else if (v4)
    dyt_f32_kernel<bf16, 4><<<grid, 256, 0, stream>>>(x, ldx, M, D, alpha, gain, shift, reinterpret_cast<bf16*>(out), ldo, alpha2, gain2,
                                                      shift2, reinterpret_cast<bf16*>(out2), ldo2);
  else
    dyt_f32_kernel<bf16, 1><<<grid, 256, 0, stream>>>(x, ldx, M, D, alpha, gain, shift, reinterpret_cast<bf16*>(out), ldo, alpha2, gain2,
                                                      shift2, reinterpret_cast<bf16*>(out2), ldo2);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_rmsnorm_gated_f32(const float* x, long long ldx, int M, int D, const float* gain, float eps, const float* gate,
                                    long long ldg, void* out, long long ldo, int out_fp32, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && gate != nullptr && out != nullptr && M >= 0 && D > 0, "lp_rmsnorm_gated_f32: bad arguments");
  if (M == 0) return 0;
  const unsigned grid = (unsigned)((M + NORM32_WARPS - 1) / NORM32_WARPS);
  const bool v4 = vec4_ok(D, {x, gate, out}, {ldx, ldg, ldo});
  if (out_fp32 && v4)
    rmsnorm_gated_f32_kernel<float, 4><<<grid, NORM32_WARPS * 32, 0, stream>>>(x, ldx, M, D, gain, eps, gate, ldg, reinterpret_cast<float*>(out), ldo);
  else if (out_fp32)
    rmsnorm_gated_f32_kernel<float, 1><<<grid, NORM32_WARPS * 32, 0, stream>>>(x, ldx, M, D, gain, eps, gate, ldg, reinterpret_cast<float*>(out), ldo);
  else if (v4)
    rmsnorm_gated_f32_kernel<bf16, 4><<<grid, NORM32_WARPS * 32, 0, stream>>>(x, ldx, M, D, gain, eps, gate, ldg, reinterpret_cast<bf16*>(out), ldo);
  else
    rmsnorm_gated_f32_kernel<bf16, 1><<<grid, NORM32_WARPS * 32, 0, stream>>>(x, ldx, M, D, gain, eps, gate, ldg, reinterpret_cast<bf16*>(out), ldo);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_gated_axpy_f32(float* x, long long ldx, const float* y, long long ldy, const float* y_bias, const float* g, long long ldg,
                                 const float* g_bias, float mult, int M, int N, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(x != nullptr && y != nullptr && M >= 0 && N > 0, "lp_gated_axpy_f32: bad arguments");
  if (M == 0) return 0;
  if (vec4_ok(N, {x, y, g}, {ldx, ldy, g != nullptr ? ldg : 0}))
    gated_axpy_f32_kernel<4><<<(unsigned)(((long long)M * (N / 4) + 255) / 256), 256, 0, stream>>>(x, ldx, y, ldy, y_bias, g, ldg, g_bias, mult, M, N);
  else
    gated_axpy_f32_kernel<1><<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, stream>>>(x, ldx, y, ldy, y_bias, g, ldg, g_bias, mult, M, N);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_depth_average_f32(const float* hist, long long layer_stride, long long ldh, const float* coef, int n, float* out,
                                    long long ldo, float* copy, long long ldc, int M, int N, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(hist != nullptr && coef != nullptr && out != nullptr && n > 0 && M >= 0 && N > 0, "lp_depth_average_f32: bad arguments");
  if (M == 0) return 0;
  if (vec4_ok(N, {hist, out, copy}, {layer_stride, ldh, ldo, copy != nullptr ? ldc : 0}))
    depth_average_f32_kernel<4><<<(unsigned)(((long long)M * (N / 4) + 255) / 256), 256, 0, stream>>>(hist, layer_stride, ldh, coef, n, out, ldo,
                                                                                                    copy, ldc, M, N);
  else
    depth_average_f32_kernel<1><<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, stream>>>(hist, layer_stride, ldh, coef, n, out, ldo,
                                                                                              copy, ldc, M, N);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_axpy_f32(float* y, long long ldy, const float* x, long long ldx, float alpha, int M, int N, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(y != nullptr && x != nullptr && M >= 0 && N > 0, "lp_axpy_f32: bad arguments");
  if (M == 0) return 0;
  axpy_f32_kernel<<<(unsigned)(((long long)M * N + 255) / 256), 256, 0, stream>>>(y, ldy, x, ldx, alpha, M, N);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}
