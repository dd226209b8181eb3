// leopard_b200 — mixture-of-experts routing for token-choice layers (scores and choices in 32-bit).
//
//   lp_moe_route     one warp per token: logits z = W_router h (fp32 accumulation over the bf16 router matrix), scores s = sigmoid(z);
//                    choice scores = s + correction (a per-expert bias that steers the choice but not the weights); experts form
//                    `n_groups` equal groups of neighbours, a group's score is the sum of its two largest choice scores, only the
//                    `keep_groups` best groups stay eligible (the others count as minus infinity); the `top` eligible experts with the
//                    largest choice scores are chosen, ties to the lower index; weights = chosen s / (sum of chosen s + 1e-20).
//                    Optionally one more row of weights gives a per-token sigmoid gate (for a shared expert).
//   lp_moe_route_softmax  the plain token-choice router on the same kernel: logits z = W_router h + bias, the `top` largest logits are
//                    chosen (ties to the lower index), weights = softmax over the chosen logits only.
//   lp_moe_route_sigmoid  the plain sigmoid router on the same kernel: the `top` largest scores sigmoid(z) are chosen and are the
//                    weights as they are (for designs that multiply an expert's INPUT by its score: lp_moe_sorted_weights puts the
//                    weights into the row space of lp_moe_align, the grouped products take them as row scales).
//   lp_moe_align     sorts the (token, choice) pairs by expert into a row space where every expert's segment is padded to whole
//                    64-row tiles (the tile of lp_linear_grouped): tile_group[tile] = expert or -1, sorted_token[row] = token or -1,
//                    pair_row[token * top + k] = the pair's row.  Sizes stay on the device: no host synchronisation.
//   lp_moe_combine   out[t] = sum_k w[t, k] y[pair_row[t, k]] (+ gate[t] * shared[t]): deterministic, no atomics on the output.
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

constexpr int MOE_MAX_EXPERTS = 512;
constexpr int ROUTE_WARPS = 8;

// eight bf16 values of a 16-byte load -> fp32 (a bf16 is the upper half of an fp32)
__device__ __forceinline__ void bf16x8_to_f32(const uint4& u, float* f) {
  f[0] = __uint_as_float(u.x << 16); f[1] = __uint_as_float(u.x & 0xffff0000u);
  f[2] = __uint_as_float(u.y << 16); f[3] = __uint_as_float(u.y & 0xffff0000u);
  f[4] = __uint_as_float(u.z << 16); f[5] = __uint_as_float(u.z & 0xffff0000u);
  f[6] = __uint_as_float(u.w << 16); f[7] = __uint_as_float(u.w & 0xffff0000u);
}

template <typename HT> __device__ __forceinline__ float moe_ld(const HT* p);
template <> __device__ __forceinline__ float moe_ld<float>(const float* p) { return *p; }
template <> __device__ __forceinline__ float moe_ld<bf16>(const bf16* p) { return __bfloat162float(*p); }

// One CTA per token: the warps share out the router rows (and the gate row), 16-byte loads of the bf16 weights when the width
// allows; then one thread makes the choice among the E scores.
template <typename HT>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const HT* __restrict__ h, long long ldh, int T, int D, const bf16* __restrict__ w_router, long long ldw, int E,
                 const float* __restrict__ correction, int n_groups, int keep_groups, int top, const bf16* __restrict__ w_gate,
                 int* __restrict__ idx_out, float* __restrict__ w_out, float* __restrict__ gate_out, int softmax_mode,
                 const float* __restrict__ logit_bias) {
  __shared__ float sc[MOE_MAX_EXPERTS];   // sigmoid scores
  __shared__ float ch[MOE_MAX_EXPERTS];   // choice scores (minus infinity once taken or not eligible)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  if (t >= T) return;
  const HT* hr = h + (long long)t * ldh;
  const bool vec = (D % 8 == 0) && (ldw % 8 == 0) && ((reinterpret_cast<uintptr_t>(w_router) & 15) == 0) &&
                   (w_gate == nullptr || (reinterpret_cast<uintptr_t>(w_gate) & 15) == 0);
  for (int e = warp; e <= E; e += ROUTE_WARPS) {
    if (e == E && w_gate == nullptr) break;
    const bf16* wr = e < E ? w_router + (long long)e * ldw : w_gate;
    float acc = 0.f;
    if (vec) {
      for (int c = lane * 8; c < D; c += 256) {
        float f[8];
        bf16x8_to_f32(*reinterpret_cast<const uint4*>(wr + c), f);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc = fmaf(moe_ld<HT>(hr + c + i), f[i], acc);
      }
    } else {
      for (int c = lane; c < D; c += 32) acc = fmaf(moe_ld<HT>(hr + c), __bfloat162float(wr[c]), acc);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    const float s = 1.0f / (1.0f + expf(-acc));
    if (lane == 0) {
      if (softmax_mode == 1) {      // the logit itself is score and choice
        sc[e] = ch[e] = acc + (logit_bias != nullptr ? logit_bias[e] : 0.f);
      } else if (e < E) {
        sc[e] = s;
        ch[e] = s + (correction != nullptr ? correction[e] : 0.f);
      } else {
        gate_out[t] = s;
      }
    }
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  if (n_groups > 1 && keep_groups < n_groups) {
    const int gs = E / n_groups;
    // group score: the sum of the two largest choice scores (of the only one when groups hold a single expert)
    float gscore[64];
    for (int g = 0; g < n_groups; ++g) {
      float a = -INFINITY, b = -INFINITY;
      for (int i = 0; i < gs; ++i) {
        const float v = ch[g * gs + i];
        if (v > a) { b = a; a = v; } else if (v > b) { b = v; }
      }
      gscore[g] = gs >= 2 ? a + b : a;
    }
    // keep the best groups: mark the others
    bool kept[64];
    for (int g = 0; g < n_groups; ++g) kept[g] = false;
    for (int k = 0; k < keep_groups; ++k) {
      int best = -1;
      for (int g = 0; g < n_groups; ++g)
        if (!kept[g] && (best < 0 || gscore[g] > gscore[best])) best = g;
      kept[best] = true;
    }
    for (int g = 0; g < n_groups; ++g)
      if (!kept[g])
        for (int i = 0; i < gs; ++i) ch[g * gs + i] = -INFINITY;
  }
  if (softmax_mode == 1) {
    float mx = -INFINITY, sum = 0.f;
    for (int k = 0; k < top; ++k) {
      int best = 0;
      for (int e = 1; e < E; ++e)
        if (ch[e] > ch[best]) best = e;
      idx_out[(long long)t * top + k] = best;
      if (k == 0) mx = sc[best];      // the first choice is the largest logit
      const float p = expf(sc[best] - mx);
      w_out[(long long)t * top + k] = p;
      sum += p;
      ch[best] = -INFINITY;
    }
    for (int k = 0; k < top; ++k) w_out[(long long)t * top + k] /= sum;
    return;
  }
  float sum = 0.f;
  for (int k = 0; k < top; ++k) {
    int best = 0;
    for (int e = 1; e < E; ++e)
      if (ch[e] > ch[best]) best = e;
    idx_out[(long long)t * top + k] = best;
    sum += sc[best];
    ch[best] = -INFINITY;   // taken; the host guarantees that the eligible experts outnumber `top`
  }
  // softmax_mode 2: the chosen scores as they are
  for (int k = 0; k < top; ++k)
    w_out[(long long)t * top + k] = sc[idx_out[(long long)t * top + k]] / (softmax_mode == 2 ? 1.0f : sum + 1e-20f);
}

__global__ void moe_sorted_weights_kernel(const int* __restrict__ pair_row, const float* __restrict__ w, int n_pairs, float* __restrict__ sorted) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n_pairs) sorted[pair_row[i]] = w[i];
}

// one CTA: counts, padded offsets, scatter
constexpr int ALIGN_THREADS = 1024;
__global__ void __launch_bounds__(ALIGN_THREADS)
moe_align_kernel(const int* __restrict__ idx, int n_pairs, int top, int E, int tile_rows, int max_tiles, int* __restrict__ tile_group,
                 int* __restrict__ sorted_token, int* __restrict__ pair_row) {
  __shared__ unsigned cnt[MOE_MAX_EXPERTS];
  __shared__ int off[MOE_MAX_EXPERTS + 1];
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) cnt[e] = 0u;
  for (int i = tid; i < max_tiles * tile_rows; i += blockDim.x) sorted_token[i] = -1;
  for (int i = tid; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
  __syncthreads();
  for (int i = tid; i < n_pairs; i += blockDim.x) pair_row[i] = (int)atomicAdd(&cnt[idx[i]], 1u);   // rank inside the expert's segment
  __syncthreads();
  if (tid == 0) {
    int o = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = o;
      const int tiles = ((int)cnt[e] + tile_rows - 1) / tile_rows;
      for (int k = 0; k < tiles; ++k) tile_group[o / tile_rows + k] = e;
      o += tiles * tile_rows;
    }
    off[E] = o;
  }
  __syncthreads();
  for (int i = tid; i < n_pairs; i += blockDim.x) {
    const int row = off[idx[i]] + pair_row[i];
    pair_row[i] = row;
    sorted_token[row] = i / top;
  }
}

__global__ void moe_combine_kernel(const float* __restrict__ y, long long ldy, const int* __restrict__ pair_row, const float* __restrict__ w,
                                   int top, const float* __restrict__ shared, long long lds, const float* __restrict__ gate,
                                   float* __restrict__ out, long long ldo, int T, int D) {
  const int t = blockIdx.x;
  if (t >= T) return;
  for (int c = threadIdx.x; c < D; c += blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)
      acc = fmaf(w != nullptr ? w[(long long)t * top + k] : 1.0f, y[(long long)pair_row[(long long)t * top + k] * ldy + c], acc);
    if (shared != nullptr) acc = fmaf(gate != nullptr ? gate[t] : 1.0f, shared[(long long)t * lds + c], acc);
    out[(long long)t * ldo + c] = acc;
  }
}

}  // namespace lp

using namespace lp;

extern "C" int lp_moe_route(const void* h, long long ldh, int h_fp32, int T, int D, const void* w_router, long long ldw, int E,
                            const float* correction, int n_groups, int keep_groups, int top, const void* w_gate, int* idx_out,
                            float* w_out, float* gate_out, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(h != nullptr && w_router != nullptr && idx_out != nullptr && w_out != nullptr, "lp_moe_route: null operand");
  LP_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "lp_moe_route: experts=%d top=%d (at most %d experts)", E, top,
             MOE_MAX_EXPERTS);
  LP_REQUIRE(n_groups >= 1 && n_groups <= 64 && E % n_groups == 0 && keep_groups >= 1 && keep_groups <= n_groups,
             "lp_moe_route: groups=%d keep=%d must divide experts=%d (at most 64 groups)", n_groups, keep_groups, E);
  LP_REQUIRE(keep_groups * (E / n_groups) >= top, "lp_moe_route: %d kept groups of %d experts cannot supply top=%d", keep_groups,
             E / n_groups, top);
  LP_REQUIRE(w_gate == nullptr || gate_out != nullptr, "lp_moe_route: gate weights without an output");
  if (T <= 0) return 0;
  const unsigned grid = (unsigned)T;
  if (h_fp32)
    moe_route_kernel<float><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const float*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, correction, n_groups, keep_groups, top, reinterpret_cast<const bf16*>(w_gate),
        idx_out, w_out, gate_out, 0, nullptr);
  else
    moe_route_kernel<bf16><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const bf16*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, correction, n_groups, keep_groups, top, reinterpret_cast<const bf16*>(w_gate),
        idx_out, w_out, gate_out, 0, nullptr);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_moe_route_softmax(const void* h, long long ldh, int h_fp32, int T, int D, const void* w_router, long long ldw, int E,
                                    const float* logit_bias, int top, int* idx_out, float* w_out, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(h != nullptr && w_router != nullptr && idx_out != nullptr && w_out != nullptr, "lp_moe_route_softmax: null operand");
  LP_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "lp_moe_route_softmax: experts=%d top=%d (at most %d experts)", E, top,
             MOE_MAX_EXPERTS);
  if (T <= 0) return 0;
  const unsigned grid = (unsigned)T;
  if (h_fp32)
    moe_route_kernel<float><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const float*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, nullptr, 1, 1, top, nullptr, idx_out, w_out, nullptr, 1, logit_bias);
  else
    moe_route_kernel<bf16><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const bf16*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, nullptr, 1, 1, top, nullptr, idx_out, w_out, nullptr, 1, logit_bias);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_moe_route_sigmoid(const void* h, long long ldh, int h_fp32, int T, int D, const void* w_router, long long ldw, int E,
                                    int top, int* idx_out, float* w_out, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(h != nullptr && w_router != nullptr && idx_out != nullptr && w_out != nullptr, "lp_moe_route_sigmoid: null operand");
  LP_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && top <= E, "lp_moe_route_sigmoid: experts=%d top=%d (at most %d experts)", E, top,
             MOE_MAX_EXPERTS);
  if (T <= 0) return 0;
  const unsigned grid = (unsigned)T;
  if (h_fp32)
    moe_route_kernel<float><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const float*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, nullptr, 1, 1, top, nullptr, idx_out, w_out, nullptr, 2, nullptr);
  else
    moe_route_kernel<bf16><<<grid, ROUTE_WARPS * 32, 0, stream>>>(reinterpret_cast<const bf16*>(h), ldh, T, D,
        reinterpret_cast<const bf16*>(w_router), ldw, E, nullptr, 1, 1, top, nullptr, idx_out, w_out, nullptr, 2, nullptr);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_moe_sorted_weights(const int* pair_row, const float* w, int n_pairs, float* sorted, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(pair_row != nullptr && w != nullptr && sorted != nullptr, "lp_moe_sorted_weights: null operand");
  if (n_pairs <= 0) return 0;
  moe_sorted_weights_kernel<<<(n_pairs + 255) / 256, 256, 0, stream>>>(pair_row, w, n_pairs, sorted);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_moe_max_tiles(int n_pairs, int E, int tile_rows) {
  const int full = (n_pairs + tile_rows - 1) / tile_rows + E;
  return full < n_pairs ? full : n_pairs;
}

extern "C" int lp_moe_align(const int* idx, int n_pairs, int top, int E, int tile_rows, int max_tiles, int* tile_group, int* sorted_token,
                            int* pair_row, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(idx != nullptr && tile_group != nullptr && sorted_token != nullptr && pair_row != nullptr, "lp_moe_align: null operand");
  LP_REQUIRE(E > 0 && E <= MOE_MAX_EXPERTS && top > 0 && tile_rows > 0, "lp_moe_align: bad sizes");
  LP_REQUIRE(max_tiles >= lp_moe_max_tiles(n_pairs, E, tile_rows), "lp_moe_align: max_tiles=%d is too small for %d pairs", max_tiles, n_pairs);
  if (n_pairs <= 0) return 0;
  moe_align_kernel<<<1, ALIGN_THREADS, 0, stream>>>(idx, n_pairs, top, E, tile_rows, max_tiles, tile_group, sorted_token, pair_row);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_moe_combine(const float* y, long long ldy, const int* pair_row, const float* w, int top, const float* shared,
                              long long lds, const float* gate, float* out, long long ldo, int T, int D, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(y != nullptr && pair_row != nullptr && out != nullptr, "lp_moe_combine: null operand");
  if (T <= 0) return 0;
  moe_combine_kernel<<<T, 128, 0, stream>>>(y, ldy, pair_row, w, top, shared, lds, gate, out, ldo, T, D);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}
