// leopard_b200 — general linear layers for the 32-bit residual-stream models (any M, N, K; fp32 or bf16 activations).
//
//   lp_linear          C[M,N] = epi(A[M,K] · W[N,K]^T): A fp32 or bf16, W bf16 (nn.Linear layout), C fp32 or bf16, accumulation in
//                      fp32 FMAs in index order of K (no tensor-core rounding: with fp32 A this is a true 32-bit product, the bf16
//                      weight is exact in fp32).  Epilogues: none, xIELU, squared relu, gated SiLU and the clamped gated unit (W =
//                      [gate rows; up rows], C has N/2 columns).  Before the epilogue every accumulator may be multiplied by a
//                      number per output row (row_scale: a router weight that multiplies an expert's INPUT is the same as one
//                      that multiplies its first products) and take a bias per weight row.  With c_accum the result is scaled
//                      and ADDED to C (the residual update of a pre-norm layer); with `gate` it is first multiplied by
//                      sigmoid(gate[m, n]) (a gated residual branch closes in the store of its last product).
//                      `batch` independent problems with element strides (per-head products of latent attention).
//                      Two kernels: a 64 x 64 x 16 shared-memory tile kernel (prefill), and a weight-streaming kernel with one warp
//                      per output column for M <= 8 rows (decode: every weight byte is read once, 16-byte loads).
//   lp_linear_grouped  the same tile kernel over row tiles that each belong to one group (expert): tile t multiplies rows
//                      [64 t, 64 t + 64) of the padded, group-sorted row space by the weight of group tile_group[t] (< 0: skip);
//                      a_rows (optional) gathers the A row of each sorted row (< 0: a padding row, computed as zero).
//
// The tcgen05 GEMM (lp_gemm_bf16) stays the matrix product of large bf16 problems; these kernels cover what it does not take:
// fp32 operands, arbitrary shapes, few rows, and row-indexed groups whose sizes are only known on the device.
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

constexpr int LIN_BM = 64, LIN_BN = 64, LIN_BK = 16, LIN_THREADS = 256;

struct LinArgs {
  const void* A; long long lda; long long a_batch;
  const bf16* W; long long ldw; long long w_batch;
  void* C; long long ldc; long long c_batch;
  int M, N, K;            // N = rows of W that are used (gated: 2 x output columns)
  int epi; float e0, e1;  // lp_linear_epi and its two constants
  int c_accum; float c_scale;   // C <- C + c_scale * epi(A W^T) instead of C <- epi(A W^T)
  const int* a_rows;      // grouped: source row of each sorted row, or NULL
  const int* tile_group;  // grouped: group of each row tile, or NULL
  const int* z_group;     // pairs (rows kernel): weight group of problem z, or NULL; problem z reads A row z / a_div and writes C row z
  int a_div;
  const float* bias;      // [N] added to the accumulators before the epilogue, or NULL
  const float* row_scale; // [rows of C] multiplies the accumulators before the bias, or NULL
  const float* gate; long long ldg;   // [rows of C, N'] pre-activations: the result is multiplied by sigmoid(gate), or NULL
};

__device__ __forceinline__ float lin_load(const float* p) { return *p; }
__device__ __forceinline__ float lin_load(const bf16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void lin_store(float* p, float v) { *p = v; }
__device__ __forceinline__ void lin_store(bf16* p, float v) { *p = __float2bfloat16(v); }

// eight bf16 values of a 16-byte load -> fp32 (a bf16 is the upper half of an fp32)
__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}

// xIELU with a = softplus(p), b = 1/2 + softplus(q):  z > 0: a z^2 + z/2;  z <= 0: b (exp(z) - 1 - z) + z/2
__device__ __forceinline__ float xielu_f(float z, float a, float b) {
  return z > 0.f ? a * z * z + 0.5f * z : b * (expm1f(z) - z) + 0.5f * z;
}
__device__ __forceinline__ float silu32_f(float z) { return z / (1.0f + expf(-z)); }

__device__ __forceinline__ float lin_epi(int epi, float v, float e0, float e1) {
  if (epi == LP_EPI_RELU2) {      // the square of relu
    const float r = fmaxf(v, 0.f);
    return r * r;
  }
  return epi == LP_EPI_XIELU ? xielu_f(v, e0, e1) : v;
}

// the two gated units: silu(g) * u, and g' sigmoid(e1 g') (u' + 1) with g' = min(g, e0), u' = clamp(u, -e0, e0)
__device__ __forceinline__ float lin_gate(int epi, float g, float u, float e0, float e1) {
  if (epi == LP_EPI_CLAMP_GLU) {
    g = fminf(g, e0);
    u = fminf(fmaxf(u, -e0), e0);
    return g / (1.0f + expf(-e1 * g)) * (u + 1.0f);
  }
  return silu32_f(g) * u;
}

// 64 x 64 output tile per CTA, 4 x 4 outputs per thread, K in steps of 16 through shared memory.  GATED: two accumulator sets, the
// second one for weight row n + N/2; the output is silu(first) * second.
template <typename AT, typename CT, bool GATED>
__global__ void __launch_bounds__(LIN_THREADS) linear_tile_kernel(LinArgs a) {
  __shared__ float As[LIN_BK][LIN_BM + 4];
  __shared__ float Ws[GATED ? 2 : 1][LIN_BK][LIN_BN + 4];
  const int tid = threadIdx.x;
  const int tile_m = blockIdx.y, tile_n = blockIdx.x, z = blockIdx.z;
  int group = 0;
  if (a.tile_group != nullptr) {
    group = a.tile_group[tile_m];
    if (group < 0) return;
  }
  const int n_out = GATED ? a.N / 2 : a.N;
  const AT* A = reinterpret_cast<const AT*>(a.A) + (long long)z * a.a_batch;
  const bf16* W = a.W + (long long)(z + group) * a.w_batch;   // grouped launches have one batch: z = 0
  CT* C = reinterpret_cast<CT*>(a.C) + (long long)z * a.c_batch;
  const int m0 = tile_m * LIN_BM, n0 = tile_n * LIN_BN;
  // loader mapping: 256 threads x 4 elements = 64 rows x 16 k
  const int lr = tid >> 2, lk = (tid & 3) * 4;
  long long a_row = -1;
  if (m0 + lr < a.M) {
    a_row = m0 + lr;
    if (a.a_rows != nullptr) a_row = a.a_rows[m0 + lr];
  }
  const int w_row = n0 + lr;
  float acc[4][4], acc2[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if (GATED) acc2[i][j] = 0.f;
    }
  const int tm = (tid >> 4) * 4, tn = (tid & 15) * 4;
  for (int k0 = 0; k0 < a.K; k0 += LIN_BK) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const int k = k0 + lk + i;
      As[lk + i][lr] = (a_row >= 0 && k < a.K) ? lin_load(A + a_row * a.lda + k) : 0.f;
      Ws[0][lk + i][lr] = (w_row < n_out && k < a.K) ? __bfloat162float(W[(long long)w_row * a.ldw + k]) : 0.f;
      if (GATED) Ws[1][lk + i][lr] = (w_row < n_out && k < a.K) ? __bfloat162float(W[(long long)(w_row + n_out) * a.ldw + k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < LIN_BK; ++kk) {
      float av[4], wv[4], wv2[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        av[i] = As[kk][tm + i];
        wv[i] = Ws[0][kk][tn + i];
        if (GATED) wv2[i] = Ws[1][kk][tn + i];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(av[i], wv[j], acc[i][j]);
          if (GATED) acc2[i][j] = fmaf(av[i], wv2[j], acc2[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int m = m0 + tm + i;
    if (m >= a.M) continue;
    const float rs = a.row_scale != nullptr ? a.row_scale[m] : 1.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tn + j;
      if (n >= n_out) continue;
      float z = acc[i][j] * rs, z2 = GATED ? acc2[i][j] * rs : 0.f;
      if (a.bias != nullptr) {
        z += a.bias[n];
        if (GATED) z2 += a.bias[n + n_out];
      }
      float v = GATED ? lin_gate(a.epi, z, z2, a.e0, a.e1) : lin_epi(a.epi, z, a.e0, a.e1);
      if (a.gate != nullptr) v /= 1.0f + expf(-a.gate[(long long)m * a.ldg + n]);
      if (a.c_accum) v = fmaf(a.c_scale, v, lin_load(C + (long long)m * a.ldc + n));
      lin_store(C + (long long)m * a.ldc + n, v);
    }
  }
}

// Few rows (M <= 8): one warp per output column, the lanes split K; the weight row is read once with 16-byte loads when K allows.
// The rows of A are staged in shared memory K-chunk by K-chunk (fp32, laid out so that the lanes' eight consecutive k of one
// 16-byte weight load fall into different banks) and shared by the CTA's eight columns.
constexpr int ROWS_MAX = 8, ROWS_WARPS = 8, ROWS_KC = 512, ROWS_LD = ROWS_KC / 8 + 1;
__device__ __forceinline__ int rows_slot(int kk) { return (kk & 7) * ROWS_LD + (kk >> 3); }
template <typename AT, typename CT, bool GATED>
__global__ void __launch_bounds__(ROWS_WARPS * 32) linear_rows_kernel(LinArgs a) {
  __shared__ float As[ROWS_MAX][8 * ROWS_LD];
  const int lane = threadIdx.x & 31;
  const int n = blockIdx.x * ROWS_WARPS + (threadIdx.x >> 5);
  const int z = blockIdx.z;
  const int n_out = GATED ? a.N / 2 : a.N;
  const bool active = n < n_out;
  const bool pairs = a.z_group != nullptr;
  const int M = pairs ? 1 : a.M;
  const AT* A = reinterpret_cast<const AT*>(a.A) + (pairs ? (long long)(z / a.a_div) * a.lda : (long long)z * a.a_batch);
  const bf16* W = a.W + (long long)(pairs ? a.z_group[z] : z) * a.w_batch;
  CT* C = reinterpret_cast<CT*>(a.C) + (pairs ? (long long)z * a.ldc : (long long)z * a.c_batch);
  const bf16* w1 = W + (long long)(active ? n : 0) * a.ldw;
  const bf16* w2 = W + (long long)(active ? n + n_out : 0) * a.ldw;
  float acc[ROWS_MAX], acc2[GATED ? ROWS_MAX : 1];
#pragma unroll
  for (int m = 0; m < ROWS_MAX; ++m) {
    acc[m] = 0.f;
    if (GATED) acc2[m] = 0.f;
  }
  const bool vec = (a.K % 8 == 0) && (a.ldw % 8 == 0) && ((reinterpret_cast<uintptr_t>(W) & 15) == 0);
  for (int k0 = 0; k0 < a.K; k0 += ROWS_KC) {
    const int kc = min(ROWS_KC, a.K - k0);
    __syncthreads();
    for (int i = threadIdx.x; i < M * kc; i += blockDim.x) {
      const int m = i / kc, kk = i % kc;
      As[m][rows_slot(kk)] = lin_load(A + (long long)m * a.lda + k0 + kk);
    }
    __syncthreads();
    if (!active) continue;
    if (vec) {
      for (int kk = lane * 8; kk < kc; kk += 256) {
        const uint4 u1 = *reinterpret_cast<const uint4*>(w1 + k0 + kk);
        uint4 u2 = u1;
        if (GATED) u2 = *reinterpret_cast<const uint4*>(w2 + k0 + kk);
        float f1[8], f2[8];
        bf16x8_to_f32(u1, f1);
        bf16x8_to_f32(u2, f2);
        const int base = kk >> 3;
#pragma unroll
        for (int m = 0; m < ROWS_MAX; ++m) {
          if (m < M) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float x = As[m][i * ROWS_LD + base];
              acc[m] = fmaf(x, f1[i], acc[m]);
              if (GATED) acc2[m] = fmaf(x, f2[i], acc2[m]);
            }
          }
        }
      }
    } else {
      for (int kk = lane; kk < kc; kk += 32) {
        const float f1 = __bfloat162float(w1[k0 + kk]);
        const float f2 = GATED ? __bfloat162float(w2[k0 + kk]) : 0.f;
#pragma unroll
        for (int m = 0; m < ROWS_MAX; ++m) {
          if (m < M) {
            const float x = As[m][rows_slot(kk)];
            acc[m] = fmaf(x, f1, acc[m]);
            if (GATED) acc2[m] = fmaf(x, f2, acc2[m]);
          }
        }
      }
    }
  }
  if (!active) return;
#pragma unroll
  for (int m = 0; m < ROWS_MAX; ++m) {
    if (m < M) {
      float s = acc[m], s2 = GATED ? acc2[m] : 0.f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        s += __shfl_xor_sync(0xffffffffu, s, o);
        if (GATED) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
      }
      if (lane == 0) {
        if (a.row_scale != nullptr) {
          const float rs = a.row_scale[pairs ? z : m];
          s *= rs;
          s2 *= rs;
        }
        if (a.bias != nullptr) {
          s += a.bias[n];
          if (GATED) s2 += a.bias[n + n_out];
        }
        float v = GATED ? lin_gate(a.epi, s, s2, a.e0, a.e1) : lin_epi(a.epi, s, a.e0, a.e1);
        if (a.gate != nullptr) v /= 1.0f + expf(-a.gate[(long long)(pairs ? z : m) * a.ldg + n]);
        if (a.c_accum) v = fmaf(a.c_scale, v, lin_load(C + (long long)m * a.ldc + n));
        lin_store(C + (long long)m * a.ldc + n, v);
      }
    }
  }
}

template <typename AT, typename CT, bool GATED>
static int launch_linear(const LinArgs& a, int batch, int m_tiles, bool allow_rows, cudaStream_t stream) {
  const int n_out = GATED ? a.N / 2 : a.N;
  if (allow_rows && a.M <= ROWS_MAX) {
    dim3 grid((n_out + ROWS_WARPS - 1) / ROWS_WARPS, 1, batch);
    linear_rows_kernel<AT, CT, GATED><<<grid, ROWS_WARPS * 32, 0, stream>>>(a);
  } else {
    dim3 grid((n_out + LIN_BN - 1) / LIN_BN, m_tiles, batch);
    linear_tile_kernel<AT, CT, GATED><<<grid, LIN_THREADS, 0, stream>>>(a);
  }
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

static int dispatch_linear(const LinArgs& a, int a_fp32, int c_fp32, int batch, int m_tiles, bool allow_rows, cudaStream_t stream) {
  const bool gated = a.epi == LP_EPI_SILU_GATE || a.epi == LP_EPI_CLAMP_GLU;
  if (a_fp32) {
    if (c_fp32) return gated ? launch_linear<float, float, true>(a, batch, m_tiles, allow_rows, stream)
                             : launch_linear<float, float, false>(a, batch, m_tiles, allow_rows, stream);
    return gated ? launch_linear<float, bf16, true>(a, batch, m_tiles, allow_rows, stream)
                 : launch_linear<float, bf16, false>(a, batch, m_tiles, allow_rows, stream);
  }
  if (c_fp32) return gated ? launch_linear<bf16, float, true>(a, batch, m_tiles, allow_rows, stream)
                           : launch_linear<bf16, float, false>(a, batch, m_tiles, allow_rows, stream);
  return gated ? launch_linear<bf16, bf16, true>(a, batch, m_tiles, allow_rows, stream)
               : launch_linear<bf16, bf16, false>(a, batch, m_tiles, allow_rows, stream);
}

}  // namespace lp

using namespace lp;

extern "C" int lp_linear(const lp_linear_desc* d, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(d != nullptr && d->A != nullptr && d->W != nullptr && d->C != nullptr, "lp_linear: null operand");
  LP_REQUIRE(d->M >= 0 && d->N > 0 && d->K > 0 && d->batch >= 1, "lp_linear: bad problem M=%d N=%d K=%d batch=%d", d->M, d->N, d->K,
             d->batch);
  LP_REQUIRE(d->epi >= LP_EPI_NONE && d->epi <= LP_EPI_CLAMP_GLU, "lp_linear: bad epilogue %d", d->epi);
  LP_REQUIRE((d->epi != LP_EPI_SILU_GATE && d->epi != LP_EPI_CLAMP_GLU) || d->N % 2 == 0, "lp_linear: the gated epilogue needs an even N (gate rows, then up rows)");
  if (d->M == 0) return 0;
  LinArgs a;
  a.A = d->A; a.lda = d->lda; a.a_batch = d->a_batch;
  a.W = reinterpret_cast<const bf16*>(d->W); a.ldw = d->ldw; a.w_batch = d->w_batch;
  a.C = d->C; a.ldc = d->ldc; a.c_batch = d->c_batch;
  a.M = d->M; a.N = d->N; a.K = d->K;
  a.epi = d->epi; a.e0 = d->epi_a; a.e1 = d->epi_b; a.c_accum = d->c_accum; a.c_scale = d->c_scale;
  a.a_rows = nullptr; a.tile_group = nullptr; a.z_group = nullptr; a.a_div = 1;
  a.bias = d->bias; a.row_scale = d->row_scale; a.gate = d->gate; a.ldg = d->ldg;
  LP_REQUIRE(d->batch == 1 || (d->bias == nullptr && d->row_scale == nullptr), "lp_linear: bias and row scale are for one problem");
  return dispatch_linear(a, d->a_fp32, d->c_fp32, d->batch, (d->M + LIN_BM - 1) / LIN_BM, true, stream);
}

// n_pairs one-row problems on the weight-streaming kernel: problem z multiplies A row z / a_div by the weight of group pair_group[z]
// (w_batch elements apart) into C row z — the expert products of a decode step, where every (token, choice) pair has its own weight.
extern "C" int lp_linear_pairs(const lp_linear_desc* d, const int* pair_group, int a_div, int n_pairs, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(d != nullptr && d->A != nullptr && d->W != nullptr && d->C != nullptr && pair_group != nullptr, "lp_linear_pairs: null operand");
  LP_REQUIRE(d->N > 0 && d->K > 0 && a_div >= 1 && n_pairs >= 0 && n_pairs <= 65535, "lp_linear_pairs: bad problem N=%d K=%d pairs=%d", d->N,
             d->K, n_pairs);
  LP_REQUIRE(d->epi >= LP_EPI_NONE && d->epi <= LP_EPI_CLAMP_GLU, "lp_linear_pairs: bad epilogue %d", d->epi);
  LP_REQUIRE((d->epi != LP_EPI_SILU_GATE && d->epi != LP_EPI_CLAMP_GLU) || d->N % 2 == 0, "lp_linear_pairs: the gated epilogue needs an even N");
  if (n_pairs == 0) return 0;
  LinArgs a;
  a.A = d->A; a.lda = d->lda; a.a_batch = 0;
  a.W = reinterpret_cast<const bf16*>(d->W); a.ldw = d->ldw; a.w_batch = d->w_batch;
  a.C = d->C; a.ldc = d->ldc; a.c_batch = 0;
  a.M = 1; a.N = d->N; a.K = d->K;
  a.epi = d->epi; a.e0 = d->epi_a; a.e1 = d->epi_b; a.c_accum = d->c_accum; a.c_scale = d->c_scale;
  a.a_rows = nullptr; a.tile_group = nullptr; a.z_group = pair_group; a.a_div = a_div;
  a.bias = d->bias; a.row_scale = d->row_scale; a.gate = d->gate; a.ldg = d->ldg;
  return dispatch_linear(a, d->a_fp32, d->c_fp32, n_pairs, 1, true, stream);
}

extern "C" int lp_linear_grouped(const lp_linear_desc* d, const int* tile_group, int n_tiles, const int* a_rows, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(d != nullptr && d->A != nullptr && d->W != nullptr && d->C != nullptr && tile_group != nullptr,
             "lp_linear_grouped: null operand");
  LP_REQUIRE(d->N > 0 && d->K > 0 && n_tiles >= 0, "lp_linear_grouped: bad problem N=%d K=%d tiles=%d", d->N, d->K, n_tiles);
  LP_REQUIRE(d->epi >= LP_EPI_NONE && d->epi <= LP_EPI_CLAMP_GLU, "lp_linear_grouped: bad epilogue %d", d->epi);
  LP_REQUIRE((d->epi != LP_EPI_SILU_GATE && d->epi != LP_EPI_CLAMP_GLU) || d->N % 2 == 0, "lp_linear_grouped: the gated epilogue needs an even N");
  if (n_tiles == 0) return 0;
  LinArgs a;
  a.A = d->A; a.lda = d->lda; a.a_batch = 0;
  a.W = reinterpret_cast<const bf16*>(d->W); a.ldw = d->ldw; a.w_batch = d->w_batch;   // w_batch = elements between groups
  a.C = d->C; a.ldc = d->ldc; a.c_batch = 0;
  a.M = n_tiles * LIN_BM; a.N = d->N; a.K = d->K;
  a.epi = d->epi; a.e0 = d->epi_a; a.e1 = d->epi_b; a.c_accum = d->c_accum; a.c_scale = d->c_scale;
  a.a_rows = a_rows; a.tile_group = tile_group; a.z_group = nullptr; a.a_div = 1;
  a.bias = d->bias; a.row_scale = d->row_scale; a.gate = d->gate; a.ldg = d->ldg;
  return dispatch_linear(a, d->a_fp32, d->c_fp32, 1, n_tiles, false, stream);
}

extern "C" int lp_linear_tile_rows(void) { return LIN_BM; }
