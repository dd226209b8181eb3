// leopard_b200 — grouped-query attention with sliding-window visibility rules over a paged fp32 key / value cache.
//
// One family of kernels serves the windowed attention layers of the layer-list language models; what differs between designs is a
// parameter of lp_window_attn_desc:
//   visibility   window (tokens j with 0 <= i - j < window), keep_first (the request's first tokens stay visible), pool (every block
//                of P tokens that lies wholly before the window is seen as ONE key / value, the mean of its cached rows)
//   scores       scale, softcap * tanh(score / softcap), sink (softmax denominator + 1)
//   projections  RMS norm of q and k per head or over the whole projection, rotation of the first rot_dims dimensions of q and k,
//                optional rotation of the values by their own position with the head output turned back by the query's position
//                (the weighted sum then depends on the distances i - j only)
//
//   mixing       talk: the softmax weights of the heads are mixed before they meet the values, weight_h <- sum_g talk[h, g] weight_g;
//                an output gate sigmoid(g) taken from the fused projection multiplies the heads' outputs
//
//   lp_window_attn_prep   one CTA per row: sums of squares per head, then every (pair | single) element of q, k, v is normalised,
//                         rotated and written: q in place, k and v into the request's page.
//   lp_window_attn_pool   one CTA per completed block: the mean of its P cached rows -> the block's row in the pooled pool.
//   lp_window_attn        one CTA per (row, group of QH query heads that share a key / value head).  Keys are walked 32 at a time by
//                         each warp: every LANE owns one key and its QH scores (q in shared memory, the key row read once for all
//                         QH heads; when dim is a multiple of 16 four lanes share the reading of a key, 64 contiguous bytes at a
//                         time), the warp agrees on the running maximum, then the 32 values are accumulated with the
//                         lanes spread over vdim (weights and row addresses broadcast through shared memory).  The CTA's warps take every W-th tile
//                         and merge their (maximum, denominator, sum) triples at the end.  All of it in fp32.
//   lp_window_attn_talk   one CTA per row and ALL heads, two passes over the visible keys in tiles: the first finds every head's
//                         softmax maximum and denominator, the second computes the scores again, normalises them, mixes them over
//                         the heads in shared memory and adds the values with the mixed weights.
//   lp_window_attn_talk_tiles  the same for prompts, a CTA per tile of 4 consecutive rows of a request and all heads.
//   lp_window_attn_tiles  the same for prompts, a CTA per tile of 2 or 4 consecutive rows of a request: the rows share every key and
//                         value row the tile reads, each (row, key) pair masked by the row's own rule.
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

struct WinArgs {
  float* qkv; long long ld; int q_off, k_off, v_off;
  int heads, kv_heads, dim, vdim;
  int norm_mode; const float* q_gain; const float* k_gain; float eps;
  const float* inv_freq; int rot_dims, rot_layout; float rot_mscale;
  const float* v_inv_freq; int v_rot_dims, v_rot_layout;
  float* cache; int page_size; const int* page_table; int max_pages;
  float* pooled; const int* pooled_table; int max_pooled_pages; int pool;
  int window, keep_first;
  float scale, softcap; int sink;
  const float* q_bias; const float* k_bias; const float* v_bias; int v_norm;
  const float* talk; int g_off;
  int chunk, kv_shared;
};

__device__ __forceinline__ float* win_token_row(const WinArgs& a, int seq, int pos) {
  const int page = a.page_table[(long long)seq * a.max_pages + pos / a.page_size];
  return a.cache + ((long long)page * a.page_size + pos % a.page_size) * (long long)(a.kv_heads * (a.dim + a.vdim));
}
__device__ __forceinline__ float* win_block_row(const WinArgs& a, int seq, int block) {
  const int page = a.pooled_table[(long long)seq * a.max_pooled_pages + block / a.page_size];
  return a.pooled + ((long long)page * a.page_size + block % a.page_size) * (long long)(a.kv_heads * (a.dim + a.vdim));
}

// the two members of rotation pair i
__device__ __forceinline__ void win_pair(int layout, int half, int i, int& d0, int& d1) {
  if (layout == LP_ROT_INTERLEAVED) {
    d0 = 2 * i;
    d1 = 2 * i + 1;
  } else {
    d0 = i;
    d1 = i + half;
  }
}

// what a query at `pos` sees, as one index space: [kept first tokens | pooled blocks | window tokens]
struct WinVisible {
  int n_keep, n_blocks, lo, count;
};
__device__ __forceinline__ WinVisible win_visible(const WinArgs& a, int pos) {
  WinVisible v;
  v.lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  if (a.chunk > 0 && (pos / a.chunk) * a.chunk > v.lo) v.lo = (pos / a.chunk) * a.chunk;      // nothing before the query's own block
  v.n_keep = a.keep_first < v.lo ? a.keep_first : v.lo;
  if (v.n_keep < 0) v.n_keep = 0;
  v.n_blocks = (a.pool > 0 && a.window > 0 && pos - a.window + 1 > 0) ? (pos - a.window + 1) / a.pool : 0;
  v.count = v.n_keep + v.n_blocks + (pos - v.lo + 1);
  return v;
}
__device__ __forceinline__ const float* win_visible_row(const WinArgs& a, const WinVisible& v, int seq, int t) {
  if (t < v.n_keep) return win_token_row(a, seq, t);
  if (t < v.n_keep + v.n_blocks) return win_block_row(a, seq, t - v.n_keep);
  return win_token_row(a, seq, v.lo + (t - v.n_keep - v.n_blocks));
}

constexpr int WIN_PREP_THREADS = 128;
__global__ void __launch_bounds__(WIN_PREP_THREADS)
window_attn_prep_kernel(WinArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos) {
  extern __shared__ float dyn_smem[];
  float* s_ss = dyn_smem;      // [heads + kv_heads] sums of squares, then the two totals
  const int r = blockIdx.x;
  if (r >= R) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, n_warps = blockDim.x >> 5;
  const int seq = row_seq[r], pos = row_pos[r];
  float* x = a.qkv + (long long)r * a.ld;
  const int kvh = a.kv_shared ? 0 : a.kv_heads;      // key / value heads this row brings (none: they are another layer's)
  const int units = a.heads + kvh;
  // biases of the projections: added in place before anything reads the row
  if (a.q_bias != nullptr || a.k_bias != nullptr || a.v_bias != nullptr) {
    if (a.q_bias != nullptr)
      for (int i = tid; i < a.heads * a.dim; i += blockDim.x) x[a.q_off + i] += a.q_bias[i];
    if (a.k_bias != nullptr && kvh)
      for (int i = tid; i < a.kv_heads * a.dim; i += blockDim.x) x[a.k_off + i] += a.k_bias[i];
    if (a.v_bias != nullptr && kvh)
      for (int i = tid; i < a.kv_heads * a.vdim; i += blockDim.x) x[a.v_off + i] += a.v_bias[i];
    __syncthreads();
  }
  float* s_vss = s_ss + units + 2;      // [kv_heads] sums of squares of the value heads
  if (a.v_norm && kvh) {
    for (int u = warp; u < a.kv_heads; u += n_warps) {
      const float* src = x + a.v_off + u * a.vdim;
      float ss = 0.f;
      for (int d = lane; d < a.vdim; d += 32) ss = fmaf(src[d], src[d], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_vss[u] = ss;
    }
    __syncthreads();
  }
  if (a.norm_mode != LP_QKNORM_NONE) {
    for (int u = warp; u < units; u += n_warps) {
      const float* src = u < a.heads ? x + a.q_off + u * a.dim : x + a.k_off + (u - a.heads) * a.dim;
      float ss = 0.f;
      for (int d = lane; d < a.dim; d += 32) ss = fmaf(src[d], src[d], ss);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (lane == 0) s_ss[u] = ss;
    }
    __syncthreads();
    if (a.norm_mode == LP_QKNORM_FULL) {
      if (tid == 0) {
        float tq = 0.f, tk = 0.f;
        for (int u = 0; u < a.heads; ++u) tq += s_ss[u];
        for (int u = a.heads; u < units; ++u) tk += s_ss[u];
        s_ss[units] = tq;
        s_ss[units + 1] = tk;
      }
      __syncthreads();
    }
  }
  float* crow = win_token_row(a, seq, pos);
  // q and k: per head rot_dims / 2 pairs and dim - rot_dims single dimensions
  const int half = a.rot_dims >> 1;
  const int per = a.dim - half;
  for (int it = tid; it < units * per; it += blockDim.x) {
    const int u = it / per, e = it % per;
    const bool is_q = u < a.heads;
    const int hl = is_q ? u : u - a.heads;      // head inside its projection
    const float* src = is_q ? x + a.q_off + hl * a.dim : x + a.k_off + hl * a.dim;
    float* dst = is_q ? x + a.q_off + hl * a.dim : crow + hl * a.dim;
    float rinv = 1.f;
    const float* gain = nullptr;
    if (a.norm_mode == LP_QKNORM_HEAD) {
      rinv = 1.0f / sqrtf(s_ss[u] / (float)a.dim + a.eps);
      gain = is_q ? a.q_gain : a.k_gain;
    } else if (a.norm_mode == LP_QKNORM_FULL) {
      rinv = 1.0f / sqrtf(s_ss[units + (is_q ? 0 : 1)] / (float)((is_q ? a.heads : a.kv_heads) * a.dim) + a.eps);
      gain = (is_q ? a.q_gain : a.k_gain) + hl * a.dim;
    }
    if (e < half) {
      int d0, d1;
      win_pair(a.rot_layout, half, e, d0, d1);
      float u0 = src[d0] * rinv, u1 = src[d1] * rinv;
      if (gain != nullptr) {
        u0 *= gain[d0];
        u1 *= gain[d1];
      }
      float s, c;
      sincosf((float)pos * a.inv_freq[e], &s, &c);
      s *= a.rot_mscale;
      c *= a.rot_mscale;
      dst[d0] = u0 * c - u1 * s;
      dst[d1] = u1 * c + u0 * s;
    } else {
      const int d = a.rot_dims + (e - half);
      float v = src[d] * rinv;
      if (gain != nullptr) v *= gain[d];
      dst[d] = v;
    }
  }
  // values: rotated over v_rot_dims by their own position when a table is given
  const int vhalf = a.v_inv_freq != nullptr ? a.v_rot_dims >> 1 : 0;
  const int vrot = 2 * vhalf;
  const int vper = a.vdim - vhalf;
  for (int it = tid; it < kvh * vper; it += blockDim.x) {
    const int g = it / vper, e = it % vper;
    const float* src = x + a.v_off + g * a.vdim;
    float* dst = crow + a.kv_heads * a.dim + g * a.vdim;
    const float vinv = a.v_norm ? 1.0f / sqrtf(s_vss[g] / (float)a.vdim + a.eps) : 1.f;      // unit RMS per value head, cached so
    if (e < vhalf) {
      int d0, d1;
      win_pair(a.v_rot_layout, vhalf, e, d0, d1);
      float s, c;
      sincosf((float)pos * a.v_inv_freq[e], &s, &c);
      const float u0 = src[d0] * vinv, u1 = src[d1] * vinv;
      dst[d0] = u0 * c - u1 * s;
      dst[d1] = u1 * c + u0 * s;
    } else {
      const int d = vrot + (e - vhalf);
      dst[d] = src[d] * vinv;
    }
  }
}

constexpr int WIN_POOL_THREADS = 128;
__global__ void __launch_bounds__(WIN_POOL_THREADS)
window_attn_pool_kernel(WinArgs a, int n_seqs, const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0) {
  const int s = blockIdx.x;
  if (s >= n_seqs) return;
  const int pos0 = seq_pos0[s], len = seq_row0[s + 1] - seq_row0[s];
  const int b = pos0 / a.pool + blockIdx.y;
  if (b >= (pos0 + len) / a.pool) return;      // block b is complete when its last token b P + P - 1 has been written
  const int roww = a.kv_heads * (a.dim + a.vdim);
  const int c = blockIdx.z * WIN_POOL_THREADS + threadIdx.x;      // one column of the row per thread, the rows in their order
  if (c >= roww) return;
  float sum = 0.f;
  for (int j = 0; j < a.pool; ++j) sum += win_token_row(a, s, b * a.pool + j)[c];
  win_block_row(a, s, b)[c] = sum / (float)a.pool;
}

template <int QH, int NV>
__global__ void __launch_bounds__(256)
window_attn_kernel(WinArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos, void* __restrict__ out, long long ldo,
                   int out_fp32) {
  extern __shared__ float dyn_smem[];
  const int r = blockIdx.x;
  if (r >= R) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, W = blockDim.x >> 5;
  const int ratio = a.heads / a.kv_heads, per_g = ratio / QH;
  const int g = blockIdx.y / per_g, h0 = g * ratio + (blockIdx.y % per_g) * QH;
  const float** row_s = reinterpret_cast<const float**>(dyn_smem);      // [W][32] cache row of each key of a warp's current tile
  float* q_s = dyn_smem + 2 * W * 32;       // [QH][dim]
  float* p_s = q_s + QH * a.dim;            // [W][QH][32] softmax weights of a warp's current tile
  float* m_s = p_s + W * QH * 32;           // [W][QH]
  float* d_s = m_s + W * QH;                // [W][QH]
  float* o_s = d_s + W * QH;                // [W][QH][vdim]
  float* f_s = o_s + W * QH * a.vdim;       // [QH][vdim] merged output before it is turned back
  const int seq = row_seq[r], pos = row_pos[r];
  const float* q = a.qkv + (long long)r * a.ld + a.q_off + (long long)h0 * a.dim;
  for (int i = tid; i < QH * a.dim; i += blockDim.x) q_s[i] = q[i];
  __syncthreads();
  const WinVisible vis = win_visible(a, pos);
  const int v_off = a.kv_heads * a.dim + g * a.vdim;
  const bool vec = (a.dim % 4 == 0) && (a.vdim % 4 == 0);      // rows and head offsets are then 16-byte aligned
  const bool quads = vec && (a.dim % 16 == 0);
  float mx[QH], den[QH], acc[QH][NV];
#pragma unroll
  for (int h = 0; h < QH; ++h) {
    // the sink is a key of score 0 without a value: warp 0 starts from it
    mx[h] = (a.sink && warp == 0) ? 0.f : -INFINITY;
    den[h] = (a.sink && warp == 0) ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[h][i] = 0.f;
  }
  float* my_p = p_s + warp * QH * 32;
  const float** my_row = row_s + warp * 32;
  for (int t0 = warp * 32; t0 < vis.count; t0 += W * 32) {
    const int t = t0 + lane;
    const bool valid = t < vis.count;
    float sc[QH];
#pragma unroll
    for (int h = 0; h < QH; ++h) sc[h] = 0.f;
    if (quads) {
      // four lanes share a key: each reads every fourth 16-byte piece of the row, so one load instruction of the warp touches 8 rows
      // of 64 contiguous bytes instead of 32 rows; four passes cover the tile's 32 keys, the partial sums meet by two shuffles
      const int piece = lane & 3, kq = lane >> 2;
      for (int i = 0; i < 4; ++i) {
        const int tk = t0 + i * 8 + kq;
        float part[QH];
#pragma unroll
        for (int h = 0; h < QH; ++h) part[h] = 0.f;
        if (tk < vis.count) {
          const float* row = win_visible_row(a, vis, seq, tk);
          if (piece == 0) my_row[i * 8 + kq] = row;
          const float* kp = row + g * a.dim + 4 * piece;
          const float* qp = q_s + 4 * piece;
          for (int d = 0; d < a.dim; d += 16) {
            const float4 k4 = *reinterpret_cast<const float4*>(kp + d);
#pragma unroll
            for (int h = 0; h < QH; ++h) {
              const float4 q4 = *reinterpret_cast<const float4*>(qp + h * a.dim + d);
              part[h] = fmaf(q4.x, k4.x, part[h]);
              part[h] = fmaf(q4.y, k4.y, part[h]);
              part[h] = fmaf(q4.z, k4.z, part[h]);
              part[h] = fmaf(q4.w, k4.w, part[h]);
            }
          }
        }
#pragma unroll
        for (int h = 0; h < QH; ++h) {
          part[h] += __shfl_xor_sync(0xffffffffu, part[h], 1);
          part[h] += __shfl_xor_sync(0xffffffffu, part[h], 2);
          if (piece == 0) my_p[h * 32 + i * 8 + kq] = part[h];
        }
      }
      __syncwarp();
#pragma unroll
      for (int h = 0; h < QH; ++h) sc[h] = my_p[h * 32 + lane];      // lane j takes key j's scores
      __syncwarp();                                                  // all read before the weights overwrite them
    } else if (valid) {
      const float* row = win_visible_row(a, vis, seq, t);
      my_row[lane] = row;      // the value pass finds the row here instead of walking the page table again
      const float* kp = row + g * a.dim;
      if (vec) {
        for (int d = 0; d < a.dim; d += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(kp + d);
#pragma unroll
          for (int h = 0; h < QH; ++h) {
            const float4 q4 = *reinterpret_cast<const float4*>(q_s + h * a.dim + d);      // one broadcast 16-byte read
            sc[h] = fmaf(q4.x, k4.x, sc[h]);
            sc[h] = fmaf(q4.y, k4.y, sc[h]);
            sc[h] = fmaf(q4.z, k4.z, sc[h]);
            sc[h] = fmaf(q4.w, k4.w, sc[h]);
          }
        }
      } else {
        for (int d = 0; d < a.dim; ++d) {
          const float kv = kp[d];
#pragma unroll
          for (int h = 0; h < QH; ++h) sc[h] = fmaf(q_s[h * a.dim + d], kv, sc[h]);
        }
      }
    }
    float corr[QH];
#pragma unroll
    for (int h = 0; h < QH; ++h) {
      float s = sc[h] * a.scale;
      if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
      if (!valid) s = -INFINITY;
      float top = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
      const float mn = fmaxf(mx[h], top);      // finite: a tile holds at least one visible key
      corr[h] = expf(mx[h] - mn);              // exp(-inf) = 0 on a warp's first tile
      const float p = valid ? expf(s - mn) : 0.f;
      float sum = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      den[h] = fmaf(den[h], corr[h], sum);
      mx[h] = mn;
      my_p[h * 32 + lane] = p;
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[h][i] *= corr[h];
    }
    __syncwarp();
    const int cnt = vis.count - t0 < 32 ? vis.count - t0 : 32;
#pragma unroll 4
    for (int jj = 0; jj < cnt; ++jj) {
      const float* vp = my_row[jj] + v_off;
      float pj[QH];
#pragma unroll
      for (int h = 0; h < QH; ++h) pj[h] = my_p[h * 32 + jj];
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int c = lane + 32 * i;
        if (c < a.vdim) {
          const float vv = vp[c];
#pragma unroll
          for (int h = 0; h < QH; ++h) acc[h][i] = fmaf(pj[h], vv, acc[h][i]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int h = 0; h < QH; ++h) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int c = lane + 32 * i;
      if (c < a.vdim) o_s[((long long)warp * QH + h) * a.vdim + c] = acc[h][i];
    }
    if (lane == 0) {
      m_s[warp * QH + h] = mx[h];
      d_s[warp * QH + h] = den[h];
    }
  }
  __syncthreads();
  for (int i = tid; i < QH * a.vdim; i += blockDim.x) {
    const int h = i / a.vdim, c = i % a.vdim;
    float top = -INFINITY;
    for (int w = 0; w < W; ++w)
      if (d_s[w * QH + h] > 0.f) top = fmaxf(top, m_s[w * QH + h]);
    float total = 0.f, v = 0.f;
    for (int w = 0; w < W; ++w) {
      if (d_s[w * QH + h] > 0.f) {      // a warp without keys contributes nothing
        const float f = expf(m_s[w * QH + h] - top);
        total = fmaf(d_s[w * QH + h], f, total);
        v = fmaf(o_s[((long long)w * QH + h) * a.vdim + c], f, v);
      }
    }
    f_s[i] = v / total;
  }
  __syncthreads();
  // turn every head's output back by the query's position (pair i by -pos * v_inv_freq[i]) and store
  const int vhalf = a.v_inv_freq != nullptr ? a.v_rot_dims >> 1 : 0;
  for (int i = tid; i < QH * a.vdim; i += blockDim.x) {
    const int h = i / a.vdim, c = i % a.vdim;
    const float* o = f_s + h * a.vdim;
    float v = o[c];
    if (c < 2 * vhalf) {
      int pair, partner;
      bool first;
      if (a.v_rot_layout == LP_ROT_INTERLEAVED) {
        pair = c >> 1;
        first = (c & 1) == 0;
        partner = first ? c + 1 : c - 1;
      } else {
        first = c < vhalf;
        pair = first ? c : c - vhalf;
        partner = first ? c + vhalf : c - vhalf;
      }
      float s, cs;
      sincosf((float)pos * a.v_inv_freq[pair], &s, &cs);
      // rotation by the negative angle: (u, v) -> (u cos + v sin, v cos - u sin)
      v = first ? o[c] * cs + o[partner] * s : o[c] * cs - o[partner] * s;
    }
    const long long at = (long long)r * ldo + (long long)(h0 + h) * a.vdim + c;
    if (out_fp32) reinterpret_cast<float*>(out)[at] = v;
    else reinterpret_cast<bf16*>(out)[at] = __float2bfloat16(v);
  }
}

// Prompts: one CTA per tile of RQ consecutive rows of one request (a piece of one of the batch's row chunks) and QH query heads of one
// key / value head, so X = RQ * QH query vectors share every key and value row that is read.  The tile walks the UNION of what its
// rows see — kept tokens of the last row, blocks of the last row, tokens from the first row's window start to the last row — and
// every (row, key) pair is masked by the row's own rule, so a row's result is the same as in the one-row kernel up to the order of
// the sums.  A key can stand in the union twice (as a kept token of a late row and as a window token of an early one); each row
// sees exactly one of the two.
template <int QH, int NV, int RQ>
__global__ void __launch_bounds__(128)
window_attn_tile_kernel(WinArgs a, int n_chunks, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_row0,
                        const int* __restrict__ chunk_len, int tiles_per_chunk, const int* __restrict__ row_pos, void* __restrict__ out,
                        long long ldo, int out_fp32) {
  extern __shared__ float dyn_smem[];
  constexpr int X = RQ * QH;
  const int c = blockIdx.x / tiles_per_chunk, sub = blockIdx.x % tiles_per_chunk;
  if (c >= n_chunks) return;
  const int len = chunk_len[c];
  if (sub * RQ >= len) return;
  const int r0 = chunk_row0[c] + sub * RQ;
  const int nrows = len - sub * RQ < RQ ? len - sub * RQ : RQ;
  const int seq = chunk_seq[c], pos0 = row_pos[r0];
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, W = blockDim.x >> 5;
  const int ratio = a.heads / a.kv_heads, per_g = ratio / QH;
  const int g = blockIdx.y / per_g, h0 = g * ratio + (blockIdx.y % per_g) * QH;
  const float** row_s = reinterpret_cast<const float**>(dyn_smem);      // [W][32]
  float* q_s = dyn_smem + 2 * W * 32;       // [X][dim]
  float* p_s = q_s + X * a.dim;             // [W][X][32]
  float* m_s = p_s + W * X * 32;            // [W][X]
  float* d_s = m_s + W * X;                 // [W][X]
  float* o_s = d_s + W * X;                 // [W][X][vdim]
  float* f_s = o_s + W * X * a.vdim;        // [X][vdim]
  for (int i = tid; i < X * a.dim; i += blockDim.x) {
    const int x = i / a.dim, d = i % a.dim, rq = x / QH, h = x % QH;
    q_s[i] = rq < nrows ? a.qkv[(long long)(r0 + rq) * a.ld + a.q_off + (long long)(h0 + h) * a.dim + d] : 0.f;
  }
  __syncthreads();
  int r_keep[RQ], r_blocks[RQ], r_lo[RQ];
#pragma unroll
  for (int rq = 0; rq < RQ; ++rq) {
    const WinVisible v = win_visible(a, pos0 + (rq < nrows ? rq : nrows - 1));
    r_keep[rq] = v.n_keep;
    r_blocks[rq] = v.n_blocks;
    r_lo[rq] = v.lo;
  }
  const WinVisible last = win_visible(a, pos0 + nrows - 1);
  WinVisible uni;      // the union, in the index space of win_visible_row
  uni.n_keep = last.n_keep;
  uni.n_blocks = last.n_blocks;
  uni.lo = r_lo[0];
  uni.count = uni.n_keep + uni.n_blocks + (pos0 + nrows - 1 - uni.lo + 1);
  const int v_off = a.kv_heads * a.dim + g * a.vdim;
  const bool quads = (a.dim % 16 == 0) && (a.vdim % 4 == 0);
  float mx[X], den[X], acc[X][NV];
#pragma unroll
  for (int x = 0; x < X; ++x) {
    mx[x] = (a.sink && warp == 0) ? 0.f : -INFINITY;
    den[x] = (a.sink && warp == 0) ? 1.f : 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i) acc[x][i] = 0.f;
  }
  float* my_p = p_s + warp * X * 32;
  const float** my_row = row_s + warp * 32;
  for (int t0 = warp * 32; t0 < uni.count; t0 += W * 32) {
    const int t = t0 + lane;
    const bool valid = t < uni.count;
    float sc[X];
#pragma unroll
    for (int x = 0; x < X; ++x) sc[x] = 0.f;
    if (quads) {
      // four lanes share a key and every lane works on two keys at a time, so that one 16-byte read of a query serves 8 products
      const int piece = lane & 3, kq = lane >> 2;
      for (int i = 0; i < 2; ++i) {
        const int ka = i * 16 + kq, kb = ka + 8;
        const bool has_a = t0 + ka < uni.count, has_b = t0 + kb < uni.count;
        float pa[X], pb[X];
#pragma unroll
        for (int x = 0; x < X; ++x) pa[x] = pb[x] = 0.f;
        if (has_a) {
          const float* row_a = win_visible_row(a, uni, seq, t0 + ka);
          const float* row_b = has_b ? win_visible_row(a, uni, seq, t0 + kb) : row_a;
          if (piece == 0) {
            my_row[ka] = row_a;
            my_row[kb] = row_b;
          }
          const float* kpa = row_a + g * a.dim + 4 * piece;
          const float* kpb = row_b + g * a.dim + 4 * piece;
          const float* qp = q_s + 4 * piece;
          for (int d = 0; d < a.dim; d += 16) {
            const float4 k4 = *reinterpret_cast<const float4*>(kpa + d);
            const float4 l4 = *reinterpret_cast<const float4*>(kpb + d);
#pragma unroll
            for (int x = 0; x < X; ++x) {
              const float4 q4 = *reinterpret_cast<const float4*>(qp + x * a.dim + d);
              pa[x] = fmaf(q4.x, k4.x, pa[x]);
              pa[x] = fmaf(q4.y, k4.y, pa[x]);
              pa[x] = fmaf(q4.z, k4.z, pa[x]);
              pa[x] = fmaf(q4.w, k4.w, pa[x]);
              pb[x] = fmaf(q4.x, l4.x, pb[x]);
              pb[x] = fmaf(q4.y, l4.y, pb[x]);
              pb[x] = fmaf(q4.z, l4.z, pb[x]);
              pb[x] = fmaf(q4.w, l4.w, pb[x]);
            }
          }
        }
#pragma unroll
        for (int x = 0; x < X; ++x) {
          pa[x] += __shfl_xor_sync(0xffffffffu, pa[x], 1);
          pa[x] += __shfl_xor_sync(0xffffffffu, pa[x], 2);
          pb[x] += __shfl_xor_sync(0xffffffffu, pb[x], 1);
          pb[x] += __shfl_xor_sync(0xffffffffu, pb[x], 2);
          if (piece == 0) {
            my_p[x * 32 + ka] = pa[x];
            my_p[x * 32 + kb] = pb[x];
          }
        }
      }
      __syncwarp();
#pragma unroll
      for (int x = 0; x < X; ++x) sc[x] = my_p[x * 32 + lane];
      __syncwarp();
    } else if (valid) {
      const float* row = win_visible_row(a, uni, seq, t);
      my_row[lane] = row;
      const float* kp = row + g * a.dim;
      for (int d = 0; d < a.dim; ++d) {
        const float kv = kp[d];
#pragma unroll
        for (int x = 0; x < X; ++x) sc[x] = fmaf(q_s[x * a.dim + d], kv, sc[x]);
      }
    }
    // which of the tile's rows see this lane's key
    const int seg = t < uni.n_keep ? 0 : (t < uni.n_keep + uni.n_blocks ? 1 : 2);
    const int idx = seg == 0 ? t : (seg == 1 ? t - uni.n_keep : uni.lo + (t - uni.n_keep - uni.n_blocks));
#pragma unroll
    for (int x = 0; x < X; ++x) {
      const int rq = x / QH;
      bool seen = valid && rq < nrows;
      if (seg == 0) seen = seen && idx < r_keep[rq];
      else if (seg == 1) seen = seen && idx < r_blocks[rq];
      else seen = seen && idx >= r_lo[rq] && idx <= pos0 + rq;
      float s = sc[x] * a.scale;
      if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
      if (!seen) s = -INFINITY;
      float top = s;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
      const float mn = fmaxf(mx[x], top);
      const float ref = mn == -INFINITY ? 0.f : mn;      // a row that has seen nothing yet, and sees nothing in this tile
      const float corr = expf(mx[x] - ref);
      const float p = seen ? expf(s - ref) : 0.f;
      float sum = p;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      den[x] = fmaf(den[x], corr, sum);
      mx[x] = mn;
      my_p[lane * X + x] = p;      // from here on the buffer holds the weights of a key side by side
#pragma unroll
      for (int i = 0; i < NV; ++i) acc[x][i] *= corr;
    }
    __syncwarp();
    const int cnt = uni.count - t0 < 32 ? uni.count - t0 : 32;
#pragma unroll 2
    for (int jj = 0; jj < cnt; ++jj) {
      const float* vp = my_row[jj] + v_off;
      float pj[X];
#pragma unroll
      for (int x4 = 0; x4 < X / 4; ++x4) {      // X is a multiple of 4: 16-byte broadcast reads
        const float4 w4 = *reinterpret_cast<const float4*>(my_p + jj * X + 4 * x4);
        pj[4 * x4] = w4.x;
        pj[4 * x4 + 1] = w4.y;
        pj[4 * x4 + 2] = w4.z;
        pj[4 * x4 + 3] = w4.w;
      }
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const int cc = lane + 32 * i;
        if (cc < a.vdim) {
          const float vv = vp[cc];
#pragma unroll
          for (int x = 0; x < X; ++x) acc[x][i] = fmaf(pj[x], vv, acc[x][i]);
        }
      }
    }
    __syncwarp();
  }
#pragma unroll
  for (int x = 0; x < X; ++x) {
#pragma unroll
    for (int i = 0; i < NV; ++i) {
      const int cc = lane + 32 * i;
      if (cc < a.vdim) o_s[((long long)warp * X + x) * a.vdim + cc] = acc[x][i];
    }
    if (lane == 0) {
      m_s[warp * X + x] = mx[x];
      d_s[warp * X + x] = den[x];
    }
  }
  __syncthreads();
  for (int i = tid; i < X * a.vdim; i += blockDim.x) {
    const int x = i / a.vdim, cc = i % a.vdim;
    float top = -INFINITY;
    for (int w = 0; w < W; ++w)
      if (d_s[w * X + x] > 0.f) top = fmaxf(top, m_s[w * X + x]);
    float total = 0.f, v = 0.f;
    for (int w = 0; w < W; ++w) {
      if (d_s[w * X + x] > 0.f) {
        const float f = expf(m_s[w * X + x] - top);
        total = fmaf(d_s[w * X + x], f, total);
        v = fmaf(o_s[((long long)w * X + x) * a.vdim + cc], f, v);
      }
    }
    f_s[i] = total > 0.f ? v / total : 0.f;      // rows past the end of the chunk have seen nothing and are not stored
  }
  __syncthreads();
  const int vhalf = a.v_inv_freq != nullptr ? a.v_rot_dims >> 1 : 0;
  for (int i = tid; i < X * a.vdim; i += blockDim.x) {
    const int x = i / a.vdim, cc = i % a.vdim, rq = x / QH, h = x % QH;
    if (rq >= nrows) continue;
    const float* o = f_s + x * a.vdim;
    float v = o[cc];
    if (cc < 2 * vhalf) {
      int pair, partner;
      bool first;
      if (a.v_rot_layout == LP_ROT_INTERLEAVED) {
        pair = cc >> 1;
        first = (cc & 1) == 0;
        partner = first ? cc + 1 : cc - 1;
      } else {
        first = cc < vhalf;
        pair = first ? cc : cc - vhalf;
        partner = first ? cc + vhalf : cc - vhalf;
      }
      float sn, cs;
      sincosf((float)(pos0 + rq) * a.v_inv_freq[pair], &sn, &cs);
      v = first ? o[cc] * cs + o[partner] * sn : o[cc] * cs - o[partner] * sn;
    }
    const long long at = (long long)(r0 + rq) * ldo + (long long)(h0 + h) * a.vdim + cc;
    if (out_fp32) reinterpret_cast<float*>(out)[at] = v;
    else reinterpret_cast<bf16*>(out)[at] = __float2bfloat16(v);
  }
}


// Talking heads: the softmax weights of all heads are mixed, weight_h(i, j) <- sum_g talk[h, g] weight_g(i, j), before head h applies
// them to the values of its own key / value head — so a row needs the NORMALISED weights of every head at every key.  One CTA per
// row (or tile of rows) and all heads; the visible keys (the same index space as above: kept tokens, pooled blocks, window) are walked twice in tiles
// of 64 to 256 keys.  Pass 1: scores of the tile for every head -> running maximum and denominator per head.  Pass 2: the same
// scores again (the same arithmetic, so the same numbers), weights = exp(score - max) / denominator, mixed over the heads in shared
// memory, then every thread adds the tile's values to the (head, value channel) sums it owns.  Nothing is rescaled in pass 2: the
// weights are final.  An output gate, when the description names one, multiplies the sums by sigmoid(g) on the way out.
constexpr int TALK_MAX_ACC = 32;      // heads * vdim <= 256 * TALK_MAX_ACC

// what the rows of a tile see: every row's own rule, and the union that the tile walks (the index space of win_visible_row)
template <int RQ>
struct TalkRows {
  int keep[RQ], blocks[RQ], lo[RQ];
  int pos0, nrows;
  WinVisible uni;
};

// scores of one tile of keys -> p_s[row][h][jj] (scaled and capped; -inf where the row does not see the key); a thread takes one key
// and up to four query heads of one key / value head, for all RQ rows, so a key is read once for the whole tile of rows.  With
// `final_w` the maxima and inverse denominators are known and the thread writes the weight exp(score - max) / denominator (0 where
// the row does not see the key).
template <int RQ>
__device__ __forceinline__ void talk_tile_scores(const WinArgs& a, const TalkRows<RQ>& tr, int seq, int t0, int cnt, int tile, int hd4,
                                                 const float* q_s, float* p_s, const float** row_s, const float* m_s, const float* linv_s,
                                                 bool final_w, int tid, int nthreads) {
  const int H = a.heads, ratio = a.heads / a.kv_heads;
  const int hgroups = (ratio + 3) / 4;      // groups of at most four query heads per key / value head
  const int cnt4 = (cnt + 3) & ~3;
  const WinVisible& uni = tr.uni;
  for (int jj = tid; jj < cnt4; jj += nthreads) row_s[jj] = win_visible_row(a, uni, seq, t0 + (jj < cnt ? jj : 0));
  __syncthreads();
  const bool vec = (a.dim % 4 == 0) && (a.vdim % 4 == 0);
  for (int it = tid; it < a.kv_heads * hgroups * cnt; it += nthreads) {
    const int jj = it % cnt, u = it / cnt;
    const int g = u / hgroups, h0 = g * ratio + (u % hgroups) * 4;
    const int nh = (g + 1) * ratio - h0 < 4 ? (g + 1) * ratio - h0 : 4;
    const float* kp = row_s[jj] + g * a.dim;
    float sc[RQ][4];
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq)
#pragma unroll
      for (int h = 0; h < 4; ++h) sc[rq][h] = 0.f;
    if (vec) {
#pragma unroll 4
      for (int d = 0; d < a.dim; d += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kp + d);
#pragma unroll
        for (int rq = 0; rq < RQ; ++rq) {
#pragma unroll
          for (int h = 0; h < 4; ++h) {
            if (h < nh) {
              const float4 q4 = *reinterpret_cast<const float4*>(q_s + rq * hd4 + (h0 + h) * a.dim + d);
              sc[rq][h] = fmaf(q4.x, k4.x, sc[rq][h]);
              sc[rq][h] = fmaf(q4.y, k4.y, sc[rq][h]);
              sc[rq][h] = fmaf(q4.z, k4.z, sc[rq][h]);
              sc[rq][h] = fmaf(q4.w, k4.w, sc[rq][h]);
            }
          }
        }
      }
    } else {
      for (int d = 0; d < a.dim; ++d) {
        const float kv = kp[d];
#pragma unroll
        for (int rq = 0; rq < RQ; ++rq)
#pragma unroll
          for (int h = 0; h < 4; ++h)
            if (h < nh) sc[rq][h] = fmaf(q_s[rq * hd4 + (h0 + h) * a.dim + d], kv, sc[rq][h]);
      }
    }
    // which of the tile's rows see this key
    const int t = t0 + jj;
    const int seg = t < uni.n_keep ? 0 : (t < uni.n_keep + uni.n_blocks ? 1 : 2);
    const int idx = seg == 0 ? t : (seg == 1 ? t - uni.n_keep : uni.lo + (t - uni.n_keep - uni.n_blocks));
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq) {
      bool seen = rq < tr.nrows;
      if (seg == 0) seen = seen && idx < tr.keep[rq];
      else if (seg == 1) seen = seen && idx < tr.blocks[rq];
      else seen = seen && idx >= tr.lo[rq] && idx <= tr.pos0 + rq;
#pragma unroll
      for (int h = 0; h < 4; ++h) {
        if (h < nh) {
          float v = sc[rq][h] * a.scale;
          if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
          if (final_w) v = seen ? expf(v - m_s[rq * H + h0 + h]) * linv_s[rq * H + h0 + h] : 0.f;
          else if (!seen) v = -INFINITY;
          p_s[(rq * H + h0 + h) * tile + jj] = v;
        }
      }
    }
  }
  __syncthreads();
}

// One CTA per tile of RQ consecutive rows of one request (RQ = 1: per row) and ALL heads; `tile` keys at a time (a multiple of 4,
// chosen by the host so that a tile's (key, head group) pairs occupy the CTA's threads).  The tile of rows walks the UNION of what
// its rows see and every (row, key) pair is masked by the row's own rule, as in the row-tile kernel above.
// Pass 2 per tile of keys: weights p_s[row][h][key] -> mixed weights w_s[key][row][h] (a thread per key, row and four output heads;
// the mixing matrix lies transposed and padded, so one 16-byte read brings four heads' factors) -> sums: a thread owns a value
// channel of one key / value head and QH query heads of it (QH = 4, 2 or 1, whichever divides the heads per key head) for every row,
// so one value read and RQ weight reads of 16, 8 or 4 bytes feed RQ * QH sums.  When the (head group, channel) units are fewer than
// the threads, `slices` threads share a unit, each taking every slices-th key, and their sums meet in shared memory at the end.
template <int QH, int NACC, int NT, int RQ>
__global__ void __launch_bounds__(NT)
window_attn_talk_kernel(WinArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos, int n_chunks,
                        const int* __restrict__ chunk_seq, const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len,
                        int tiles_per_chunk, int tile, int slices, void* __restrict__ out, long long ldo, int out_fp32) {
  extern __shared__ float dyn_smem[];
  int r0, seq;
  TalkRows<RQ> tr;
  if (RQ == 1) {
    r0 = blockIdx.x;
    if (r0 >= R) return;
    tr.nrows = 1;
    seq = row_seq[r0];
  } else {
    const int c = blockIdx.x / tiles_per_chunk, sub = blockIdx.x % tiles_per_chunk;
    if (c >= n_chunks) return;
    const int len = chunk_len[c];
    if (sub * RQ >= len) return;
    r0 = chunk_row0[c] + sub * RQ;
    tr.nrows = len - sub * RQ < RQ ? len - sub * RQ : RQ;
    seq = chunk_seq[c];
  }
  tr.pos0 = row_pos[r0];
  const int nrows = tr.nrows;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  constexpr int n_warps = NT / 32;
  const int H = a.heads, ratio = a.heads / a.kv_heads, Hp = (H + 3) & ~3, hg4 = Hp >> 2, hd4 = (H * a.dim + 3) & ~3;
  const float** row_s = reinterpret_cast<const float**>(dyn_smem);      // [tile] cache row of each key of the tile
  float* q_s = dyn_smem + 2 * tile;             // [RQ][H][dim]
  float* p_s = q_s + RQ * hd4;                  // [RQ][H][tile] scores (pass 1), weights (pass 2)
  float* w_s = p_s + RQ * H * tile;             // [tile][RQ][Hp] mixed weights
  float* t_s = w_s + RQ * Hp * tile;            // [H][Hp] the mixing matrix, transposed: t_s[g][h] = talk[h][g]
  float* m_s = t_s + H * Hp;                    // [RQ][H] maxima
  float* l_s = m_s + RQ * H;                    // [RQ][H] denominators, then their inverses
  float* red_s = l_s + RQ * H;                  // [slices][units][RQ][QH] partial sums, when slices > 1
  for (int i = tid; i < RQ * H * a.dim; i += NT) {
    const int rq = i / (H * a.dim), e = i % (H * a.dim);
    q_s[rq * hd4 + e] = rq < nrows ? a.qkv[(long long)(r0 + rq) * a.ld + a.q_off + e] : 0.f;
  }
  for (int i = tid; i < H * Hp; i += NT) {
    const int g = i / Hp, h = i % Hp;
    t_s[i] = h < H ? a.talk[h * H + g] : 0.f;
  }
  for (int i = tid; i < RQ * H; i += NT) {      // the sink is a key of score 0 without a value
    m_s[i] = a.sink ? 0.f : -INFINITY;
    l_s[i] = a.sink ? 1.f : 0.f;
  }
#pragma unroll
  for (int rq = 0; rq < RQ; ++rq) {
    const WinVisible v = win_visible(a, tr.pos0 + (rq < nrows ? rq : nrows - 1));
    tr.keep[rq] = v.n_keep;
    tr.blocks[rq] = v.n_blocks;
    tr.lo[rq] = v.lo;
  }
  {
    const WinVisible last = win_visible(a, tr.pos0 + nrows - 1);
    tr.uni.n_keep = last.n_keep;
    tr.uni.n_blocks = last.n_blocks;
    tr.uni.lo = tr.lo[0];
    tr.uni.count = last.n_keep + last.n_blocks + (tr.pos0 + nrows - 1 - tr.lo[0] + 1);
  }
  const int count = tr.uni.count;
  __syncthreads();
  // pass 1: maxima and denominators
  for (int t0 = 0; t0 < count; t0 += tile) {
    const int cnt = count - t0 < tile ? count - t0 : tile;
    talk_tile_scores<RQ>(a, tr, seq, t0, cnt, tile, hd4, q_s, p_s, row_s, nullptr, nullptr, false, tid, NT);
    for (int x = warp; x < nrows * H; x += n_warps) {      // x = row * H + head
      float top = -INFINITY;
      for (int jj = lane; jj < cnt; jj += 32) top = fmaxf(top, p_s[x * tile + jj]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) top = fmaxf(top, __shfl_xor_sync(0xffffffffu, top, o));
      const float mn = fmaxf(m_s[x], top);
      const float ref = mn == -INFINITY ? 0.f : mn;      // a row that has seen nothing yet, and sees nothing in this tile
      float sum = 0.f;
      for (int jj = lane; jj < cnt; jj += 32) sum += expf(p_s[x * tile + jj] - ref);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
      __syncwarp();
      if (lane == 0) {
        l_s[x] = fmaf(l_s[x], expf(m_s[x] - ref), sum);      // exp(-inf) = 0 on the first tile
        m_s[x] = mn;
      }
    }
    __syncthreads();
  }
  for (int i = tid; i < nrows * H; i += NT) l_s[i] = 1.0f / l_s[i];
  __syncthreads();
  // pass 2: final weights, mixed, times the values
  float acc[NACC][RQ][QH];
#pragma unroll
  for (int i = 0; i < NACC; ++i)
#pragma unroll
    for (int rq = 0; rq < RQ; ++rq)
#pragma unroll
      for (int x = 0; x < QH; ++x) acc[i][rq][x] = 0.f;
  const int nqg = ratio / QH;                       // query-head groups per key / value head
  const int units = a.kv_heads * nqg * a.vdim;      // (key / value head, query group, channel)
  const int v_base = a.kv_heads * a.dim;
  for (int t0 = 0; t0 < count; t0 += tile) {
    const int cnt = count - t0 < tile ? count - t0 : tile;
    talk_tile_scores<RQ>(a, tr, seq, t0, cnt, tile, hd4, q_s, p_s, row_s, m_s, l_s, true, tid, NT);
    for (int it = tid; it < hg4 * RQ * cnt; it += NT) {
      const int hq = it % hg4, rq = (it / hg4) % RQ, jj = it / (hg4 * RQ);
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      const float* pp = p_s + rq * H * tile + jj;
      for (int g = 0; g < H; ++g) {
        const float p = pp[g * tile];
        const float4 t4 = *reinterpret_cast<const float4*>(t_s + g * Hp + 4 * hq);
        v.x = fmaf(t4.x, p, v.x);
        v.y = fmaf(t4.y, p, v.y);
        v.z = fmaf(t4.z, p, v.z);
        v.w = fmaf(t4.w, p, v.w);
      }
      *reinterpret_cast<float4*>(w_s + (jj * RQ + rq) * Hp + 4 * hq) = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
      const int e = tid + i * NT;
      if (e < units * slices) {
        const int sl = e / units, u = e % units;
        const int c = u % a.vdim, gq = u / a.vdim;      // gq = g * nqg + query group, so its first head is gq * QH
        const int off = v_base + (gq / nqg) * a.vdim + c;
        const float* wh = w_s + gq * QH;
#pragma unroll(RQ == 1 ? 8 : 4)      // that many value reads in flight per thread
        for (int jj = sl; jj < cnt; jj += slices) {
          const float v = row_s[jj][off];
#pragma unroll
          for (int rq = 0; rq < RQ; ++rq) {
            const float* wp = wh + (jj * RQ + rq) * Hp;
            if (QH == 4) {
              const float4 w4 = *reinterpret_cast<const float4*>(wp);
              acc[i][rq][0] = fmaf(w4.x, v, acc[i][rq][0]);
              acc[i][rq][1 % QH] = fmaf(w4.y, v, acc[i][rq][1 % QH]);
              acc[i][rq][2 % QH] = fmaf(w4.z, v, acc[i][rq][2 % QH]);
              acc[i][rq][3 % QH] = fmaf(w4.w, v, acc[i][rq][3 % QH]);
            } else if (QH == 2) {
              const float2 w2 = *reinterpret_cast<const float2*>(wp);
              acc[i][rq][0] = fmaf(w2.x, v, acc[i][rq][0]);
              acc[i][rq][1 % QH] = fmaf(w2.y, v, acc[i][rq][1 % QH]);
            } else {
              acc[i][rq][0] = fmaf(wp[0], v, acc[i][rq][0]);
            }
          }
        }
      }
    }
    __syncthreads();
  }
  if (slices > 1) {      // NACC is 1 here: every thread holds one unit's sums over its keys
    if (tid < units * slices) {
#pragma unroll
      for (int rq = 0; rq < RQ; ++rq)
#pragma unroll
        for (int x = 0; x < QH; ++x) red_s[(tid * RQ + rq) * QH + x] = acc[0][rq][x];
    }
    __syncthreads();
    if (tid < units) {
#pragma unroll
      for (int rq = 0; rq < RQ; ++rq)
#pragma unroll
        for (int x = 0; x < QH; ++x) {
          float v = 0.f;
          for (int sl = 0; sl < slices; ++sl) v += red_s[((sl * units + tid) * RQ + rq) * QH + x];
          acc[0][rq][x] = v;
        }
    }
  }
#pragma unroll
  for (int i = 0; i < NACC; ++i) {
    const int u = tid + i * NT;
    if (u < units) {
      const int c = u % a.vdim, gq = u / a.vdim;
#pragma unroll
      for (int rq = 0; rq < RQ; ++rq) {
        if (rq < nrows) {
          const float* gate = a.g_off >= 0 ? a.qkv + (long long)(r0 + rq) * a.ld + a.g_off : nullptr;
#pragma unroll
          for (int x = 0; x < QH; ++x) {
            const int e = (gq * QH + x) * a.vdim + c;
            float v = acc[i][rq][x];
            if (gate != nullptr) v *= 1.0f / (1.0f + expf(-gate[e]));
            const long long at = (long long)(r0 + rq) * ldo + e;
            if (out_fp32) reinterpret_cast<float*>(out)[at] = v;
            else reinterpret_cast<bf16*>(out)[at] = __float2bfloat16(v);
          }
        }
      }
    }
  }
}

static size_t talk_smem_bytes(int heads, int dim, int tile, int rq, int red_floats) {
  const size_t hp = ((size_t)heads + 3) & ~(size_t)3;
  return (2 * (size_t)tile + rq * (((size_t)heads * dim + 3) & ~(size_t)3) + rq * (size_t)heads * tile + rq * hp * tile + (size_t)heads * hp +
          2 * rq * (size_t)heads + (size_t)red_floats) * sizeof(float);
}

struct TalkChunks {
  int n_chunks;
  const int *seq, *row0, *len;
};

// the dynamic shared-memory limit is raised once per instantiation, and only when a launch needs it (no runtime call on the steady
// path, so the steady path can be captured into a CUDA graph).  0: launched; 1: a tile of RQ > 1 rows does not fit shared memory.
template <int QH, int NACC, int NT, int RQ>
static int launch_window_attn_talk(const WinArgs& a, int R, const int* row_seq, const int* row_pos, const TalkChunks& ch, void* out,
                                   long long ldo, int out_fp32, cudaStream_t stream) {
  const int n_units = a.heads / QH * a.vdim;
  const int slices = n_units < NT ? NT / n_units : 1;
  const int red = slices > 1 ? NT * RQ * QH : 0;
  // enough keys a tile that its (key, group of four heads) pairs give every thread one, within shared memory
  const int units = a.kv_heads * ((a.heads / a.kv_heads + 3) / 4);
  int tile = 64;
  while (tile < 256 && units * tile < NT && talk_smem_bytes(a.heads, a.dim, 2 * tile, RQ, red) <= 96 * 1024) tile *= 2;
  while (tile > 16 && talk_smem_bytes(a.heads, a.dim, tile, RQ, red) > 200 * 1024) tile /= 2;
  const size_t smem = talk_smem_bytes(a.heads, a.dim, tile, RQ, red);
  if (RQ > 1 && smem > 112 * 1024) return 1;      // two CTAs a multiprocessor
  LP_REQUIRE(smem <= 200 * 1024, "lp_window_attn_talk: heads=%d dim=%d do not fit shared memory", a.heads, a.dim);
  static size_t have = 48 * 1024;
  if (smem > have) {
    LP_CHECK_CUDA(cudaFuncSetAttribute(window_attn_talk_kernel<QH, NACC, NT, RQ>, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    have = 200 * 1024;
  }
  int grid = R, tiles = 0;
  if (RQ > 1) {
    const int longest = R < LP_RETENTION_CHUNK ? R : LP_RETENTION_CHUNK;      // no chunk has more rows than the step or the chunk size
    tiles = (longest + RQ - 1) / RQ;
    grid = ch.n_chunks * tiles;
  }
  window_attn_talk_kernel<QH, NACC, NT, RQ><<<grid, NT, smem, stream>>>(a, R, row_seq, row_pos, ch.n_chunks, ch.seq, ch.row0, ch.len, tiles,
                                                                        tile, slices, out, ldo, out_fp32);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

// the instantiation whose threads hold the fewest sums that still cover all (head group, channel) units; with chunk tables
// (prompts and portions) tiles of TALK_RQ rows where a thread's sums stay few, else (and for one-token steps) a CTA per row
constexpr int TALK_RQ = 4;
template <int QH, int NT>
static int pick_window_attn_talk(const WinArgs& a, int R, const int* row_seq, const int* row_pos, const TalkChunks& ch, void* out, long long ldo,
                                 int out_fp32, cudaStream_t stream) {
  const int per_thread = (a.heads / QH * a.vdim + NT - 1) / NT;
  if constexpr (NT == 256) {
   if (ch.n_chunks > 0 && per_thread * QH <= 8) {
    int rc;
    if (per_thread <= 1) rc = launch_window_attn_talk<QH, 1, NT, TALK_RQ>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
    else if (per_thread <= 2) rc = launch_window_attn_talk<QH, 2, NT, TALK_RQ>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
    else rc = launch_window_attn_talk<QH, 8 / QH, NT, TALK_RQ>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
    if (rc != 1) return rc;
   }
  }
  if (per_thread <= 1) return launch_window_attn_talk<QH, 1, NT, 1>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  if (per_thread <= 2) return launch_window_attn_talk<QH, 2, NT, 1>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  if (per_thread <= 8) return launch_window_attn_talk<QH, 8, NT, 1>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  if (per_thread <= 32 / QH) return launch_window_attn_talk<QH, 32 / QH, NT, 1>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  LP_REQUIRE(false, "lp_window_attn_talk: heads * vdim = %d is more than %d threads hold", a.heads * a.vdim, NT);
  return 1;
}

static int fill_win(WinArgs& a, const lp_window_attn_desc* d, bool need_q) {
  LP_REQUIRE(d != nullptr && d->cache != nullptr && d->page_table != nullptr, "lp_window_attn: null operand");
  LP_REQUIRE(!need_q || d->qkv != nullptr, "lp_window_attn: null projection");
  LP_REQUIRE(d->heads > 0 && d->kv_heads > 0 && d->heads % d->kv_heads == 0 && d->dim > 0 && d->vdim > 0,
             "lp_window_attn: bad sizes heads=%d kv_heads=%d dim=%d vdim=%d", d->heads, d->kv_heads, d->dim, d->vdim);
  LP_REQUIRE(d->page_size > 0 && d->max_pages > 0, "lp_window_attn: bad page table");
  LP_REQUIRE(d->rot_dims >= 0 && d->rot_dims <= d->dim && d->rot_dims % 2 == 0, "lp_window_attn: rot_dims=%d must be even and <= dim=%d",
             d->rot_dims, d->dim);
  LP_REQUIRE(d->rot_dims == 0 || d->inv_freq != nullptr, "lp_window_attn: rotation without a frequency table");
  LP_REQUIRE(d->v_inv_freq == nullptr || (d->v_rot_dims >= 0 && d->v_rot_dims <= d->vdim && d->v_rot_dims % 2 == 0),
             "lp_window_attn: v_rot_dims=%d must be even and <= vdim=%d", d->v_rot_dims, d->vdim);
  LP_REQUIRE(d->norm_mode >= LP_QKNORM_NONE && d->norm_mode <= LP_QKNORM_FULL, "lp_window_attn: bad norm mode %d", d->norm_mode);
  LP_REQUIRE((d->q_gain != nullptr) == (d->k_gain != nullptr), "lp_window_attn: one norm gain without the other");
  LP_REQUIRE(d->norm_mode != LP_QKNORM_NONE || d->q_gain == nullptr, "lp_window_attn: gains without a norm");
  LP_REQUIRE(d->pool >= 0 && (d->pool == 0 || (d->pooled != nullptr && d->pooled_table != nullptr && d->max_pooled_pages > 0)),
             "lp_window_attn: pooled blocks without their pool");
  LP_REQUIRE(d->keep_first >= 0, "lp_window_attn: keep_first < 0");
  a.qkv = d->qkv; a.ld = d->ld; a.q_off = d->q_off; a.k_off = d->k_off; a.v_off = d->v_off;
  a.heads = d->heads; a.kv_heads = d->kv_heads; a.dim = d->dim; a.vdim = d->vdim;
  a.norm_mode = d->norm_mode; a.q_gain = d->q_gain; a.k_gain = d->k_gain; a.eps = d->eps;
  a.inv_freq = d->inv_freq; a.rot_dims = d->rot_dims; a.rot_layout = d->rot_layout; a.rot_mscale = d->rot_mscale;
  a.v_inv_freq = d->v_inv_freq; a.v_rot_dims = d->v_rot_dims; a.v_rot_layout = d->v_rot_layout;
  a.cache = d->cache; a.page_size = d->page_size; a.page_table = d->page_table; a.max_pages = d->max_pages;
  a.pooled = d->pooled; a.pooled_table = d->pooled_table; a.max_pooled_pages = d->max_pooled_pages; a.pool = d->pool;
  a.window = d->window; a.keep_first = d->keep_first;
  a.chunk = d->chunk; a.kv_shared = d->kv_shared;
  LP_REQUIRE(d->chunk >= 0, "lp_window_attn: chunk < 0");
  LP_REQUIRE(d->chunk == 0 || (d->keep_first == 0 && d->pool == 0), "lp_window_attn: block-local visibility with kept tokens or pooled blocks is not supported");
  a.scale = d->scale; a.softcap = d->softcap; a.sink = d->sink;
  a.q_bias = d->q_bias; a.k_bias = d->k_bias; a.v_bias = d->v_bias; a.v_norm = d->v_norm;
  a.talk = d->talk; a.g_off = d->g_off;
  return 0;
}

constexpr int WIN_MAX_DIM = 256;
constexpr int WIN_SPLIT_ROWS = 16;      // up to this many rows (decoding) a CTA has 8 warps, else 4

static size_t win_smem_floats(int qh, int w, int dim, int vdim) {
  return 2 * (size_t)w * 32 + (size_t)qh * dim + (size_t)w * qh * 32 + 2 * (size_t)w * qh + (size_t)w * qh * vdim + (size_t)qh * vdim;
}

template <int QH>
static int launch_window_attn(const WinArgs& a, int R, const int* row_seq, const int* row_pos, void* out, long long ldo, int out_fp32,
                              cudaStream_t stream) {
  int warps = R <= WIN_SPLIT_ROWS ? 8 : 4;
  while (warps > 1 && win_smem_floats(QH, warps, a.dim, a.vdim) * sizeof(float) > 48 * 1024) warps >>= 1;
  const size_t smem = win_smem_floats(QH, warps, a.dim, a.vdim) * sizeof(float);
  LP_REQUIRE(smem <= 48 * 1024, "lp_window_attn: dim=%d vdim=%d do not fit shared memory", a.dim, a.vdim);
  const dim3 grid(R, a.kv_heads * (a.heads / a.kv_heads / QH));
  const int nv = (a.vdim + 31) / 32;
  if (nv <= 1) window_attn_kernel<QH, 1><<<grid, warps * 32, smem, stream>>>(a, R, row_seq, row_pos, out, ldo, out_fp32);
  else if (nv <= 2) window_attn_kernel<QH, 2><<<grid, warps * 32, smem, stream>>>(a, R, row_seq, row_pos, out, ldo, out_fp32);
  else if (nv <= 4) window_attn_kernel<QH, 4><<<grid, warps * 32, smem, stream>>>(a, R, row_seq, row_pos, out, ldo, out_fp32);
  else window_attn_kernel<QH, 8><<<grid, warps * 32, smem, stream>>>(a, R, row_seq, row_pos, out, ldo, out_fp32);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

static size_t win_tile_smem_floats(int x, int w, int dim, int vdim) {
  return 2 * (size_t)w * 32 + (size_t)x * dim + (size_t)w * x * 32 + 2 * (size_t)w * x + (size_t)w * x * vdim + (size_t)x * vdim;
}

// 0: launched; 1: the sizes do not fit the tile kernel's shared memory (the caller takes the one-row kernel)
template <int QH, int RQ>
static int launch_window_attn_tiles(const WinArgs& a, int R, int n_chunks, const int* chunk_seq, const int* chunk_row0, const int* chunk_len,
                                    const int* row_pos, void* out, long long ldo, int out_fp32, cudaStream_t stream) {
  int warps = 4;
  while (warps > 1 && win_tile_smem_floats(QH * RQ, warps, a.dim, a.vdim) * sizeof(float) > 48 * 1024) warps >>= 1;
  const size_t smem = win_tile_smem_floats(QH * RQ, warps, a.dim, a.vdim) * sizeof(float);
  if (smem > 48 * 1024) return 1;
  const int longest = R < LP_RETENTION_CHUNK ? R : LP_RETENTION_CHUNK;      // no chunk has more rows than the step or the chunk size
  const int tiles = (longest + RQ - 1) / RQ;
  const dim3 grid(n_chunks * tiles, a.kv_heads * (a.heads / a.kv_heads / QH));
  const int nv = (a.vdim + 31) / 32;
  if (nv <= 1) window_attn_tile_kernel<QH, 1, RQ><<<grid, warps * 32, smem, stream>>>(a, n_chunks, chunk_seq, chunk_row0, chunk_len, tiles, row_pos, out, ldo, out_fp32);
  else if (nv <= 2) window_attn_tile_kernel<QH, 2, RQ><<<grid, warps * 32, smem, stream>>>(a, n_chunks, chunk_seq, chunk_row0, chunk_len, tiles, row_pos, out, ldo, out_fp32);
  else if (nv <= 4) window_attn_tile_kernel<QH, 4, RQ><<<grid, warps * 32, smem, stream>>>(a, n_chunks, chunk_seq, chunk_row0, chunk_len, tiles, row_pos, out, ldo, out_fp32);
  else return 1;      // value heads wider than 128 keep too many sums per lane for a tile of rows
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

}  // namespace lp

using namespace lp;

extern "C" int lp_window_attn_prep(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  WinArgs a;
  if (int rc = fill_win(a, d, true)) return rc;
  LP_REQUIRE(row_seq != nullptr && row_pos != nullptr, "lp_window_attn_prep: null operand");
  if (R <= 0) return 0;
  const size_t smem = (size_t)(d->heads + 2 * d->kv_heads + 2) * sizeof(float);
  LP_REQUIRE(smem <= 48 * 1024, "lp_window_attn_prep: too many heads");
  window_attn_prep_kernel<<<R, WIN_PREP_THREADS, smem, stream>>>(a, R, row_seq, row_pos);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_window_attn_pool(const lp_window_attn_desc* d, int n_seqs, const int* seq_row0, const int* seq_pos0, int max_new_blocks,
                                   void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  WinArgs a;
  if (int rc = fill_win(a, d, false)) return rc;
  LP_REQUIRE(d->pool > 0 && seq_row0 != nullptr && seq_pos0 != nullptr, "lp_window_attn_pool: no pooled blocks in this description");
  if (n_seqs <= 0 || max_new_blocks <= 0) return 0;
  LP_REQUIRE(max_new_blocks <= 65535, "lp_window_attn_pool: %d blocks per request in one step", max_new_blocks);
  const int roww = d->kv_heads * (d->dim + d->vdim);
  window_attn_pool_kernel<<<dim3(n_seqs, max_new_blocks, (roww + WIN_POOL_THREADS - 1) / WIN_POOL_THREADS), WIN_POOL_THREADS, 0, stream>>>(
      a, n_seqs, seq_row0, seq_pos0);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_window_attn(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, void* out, long long ldo,
                              int out_fp32, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  WinArgs a;
  if (int rc = fill_win(a, d, true)) return rc;
  LP_REQUIRE(out != nullptr && row_seq != nullptr && row_pos != nullptr, "lp_window_attn: null operand");
  LP_REQUIRE(d->dim <= WIN_MAX_DIM && d->vdim <= WIN_MAX_DIM, "lp_window_attn: dim=%d / vdim=%d > %d is not instantiated", d->dim, d->vdim,
             WIN_MAX_DIM);
  if (R <= 0) return 0;
  const int ratio = d->heads / d->kv_heads;
  if (ratio % 4 == 0) return launch_window_attn<4>(a, R, row_seq, row_pos, out, ldo, out_fp32, stream);
  if (ratio % 2 == 0) return launch_window_attn<2>(a, R, row_seq, row_pos, out, ldo, out_fp32, stream);
  return launch_window_attn<1>(a, R, row_seq, row_pos, out, ldo, out_fp32, stream);
}

static int window_attn_talk(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, const TalkChunks& ch, void* out,
                            long long ldo, int out_fp32, cudaStream_t stream) {
  WinArgs a;
  if (int rc = fill_win(a, d, true)) return rc;
  LP_REQUIRE(out != nullptr && row_seq != nullptr && row_pos != nullptr && d->talk != nullptr, "lp_window_attn_talk: null operand");
  LP_REQUIRE(d->v_inv_freq == nullptr, "lp_window_attn_talk: rotated values are not mixed here");
  if (R <= 0) return 0;
  const int n_out = d->heads * d->vdim;
  LP_REQUIRE(n_out <= 256 * TALK_MAX_ACC, "lp_window_attn_talk: heads * vdim = %d > %d", n_out, 256 * TALK_MAX_ACC);
  const int ratio = d->heads / d->kv_heads;
  const int qh = ratio % 4 == 0 ? 4 : ratio % 2 == 0 ? 2 : 1;
  if (ch.n_chunks == 0 && R <= WIN_SPLIT_ROWS && n_out / qh >= 256) {      // few rows (decoding) of heads wide enough: 1024 threads a row
    if (qh == 4) return pick_window_attn_talk<4, 1024>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
    if (qh == 2) return pick_window_attn_talk<2, 1024>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
    return pick_window_attn_talk<1, 1024>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  }
  if (qh == 4) return pick_window_attn_talk<4, 256>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  if (qh == 2) return pick_window_attn_talk<2, 256>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
  return pick_window_attn_talk<1, 256>(a, R, row_seq, row_pos, ch, out, ldo, out_fp32, stream);
}

// one-token steps (and any rows without chunk tables): a CTA per row
extern "C" int lp_window_attn_talk(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, void* out, long long ldo,
                                   int out_fp32, void* stream_) {
  return window_attn_talk(d, R, row_seq, row_pos, TalkChunks{0, nullptr, nullptr, nullptr}, out, ldo, out_fp32,
                          reinterpret_cast<cudaStream_t>(stream_));
}

// prompts and portions: the rows come as chunks of consecutive rows of one request, and tiles of rows share the keys they read
extern "C" int lp_window_attn_talk_tiles(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, int n_chunks,
                                         const int* chunk_seq, const int* chunk_row0, const int* chunk_len, void* out, long long ldo,
                                         int out_fp32, void* stream_) {
  LP_REQUIRE(n_chunks <= 0 || (chunk_seq != nullptr && chunk_row0 != nullptr && chunk_len != nullptr), "lp_window_attn_talk_tiles: null operand");
  return window_attn_talk(d, R, row_seq, row_pos, TalkChunks{n_chunks > 0 ? n_chunks : 0, chunk_seq, chunk_row0, chunk_len}, out, ldo, out_fp32,
                          reinterpret_cast<cudaStream_t>(stream_));
}

extern "C" int lp_window_attn_tiles(const lp_window_attn_desc* d, int R, const int* row_seq, const int* row_pos, int n_chunks,
                                    const int* chunk_seq, const int* chunk_row0, const int* chunk_len, void* out, long long ldo,
                                    int out_fp32, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  WinArgs a;
  if (int rc = fill_win(a, d, true)) return rc;
  LP_REQUIRE(out != nullptr && row_seq != nullptr && row_pos != nullptr && chunk_seq != nullptr && chunk_row0 != nullptr && chunk_len != nullptr,
             "lp_window_attn_tiles: null operand");
  LP_REQUIRE(d->dim <= WIN_MAX_DIM && d->vdim <= WIN_MAX_DIM, "lp_window_attn_tiles: dim=%d / vdim=%d > %d is not instantiated", d->dim,
             d->vdim, WIN_MAX_DIM);
  if (R <= 0 || n_chunks <= 0) return 0;
  const int ratio = d->heads / d->kv_heads;
  int rc;
  if (ratio % 4 == 0) rc = launch_window_attn_tiles<4, 2>(a, R, n_chunks, chunk_seq, chunk_row0, chunk_len, row_pos, out, ldo, out_fp32, stream);
  else if (ratio % 2 == 0) rc = launch_window_attn_tiles<2, 4>(a, R, n_chunks, chunk_seq, chunk_row0, chunk_len, row_pos, out, ldo, out_fp32, stream);
  else rc = launch_window_attn_tiles<1, 4>(a, R, n_chunks, chunk_seq, chunk_row0, chunk_len, row_pos, out, ldo, out_fp32, stream);
  if (rc == 1) return lp_window_attn(d, R, row_seq, row_pos, out, ldo, out_fp32, stream_);
  return rc;
}
