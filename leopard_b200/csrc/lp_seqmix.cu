// leopard_b200 — sequence mixers with 32-bit scores and state, over packed batches of requests (prefill rows or one row per request).
//
//   Rotary positions     angle = position * inv_freq[i] in fp32, accurate sincosf; two pairings: LP_ROT_HALF (i with i + dims/2) and
//                        LP_ROT_INTERLEAVED (2i with 2i + 1); both cos and sin carry a magnitude factor (frequency-rescaled tables such as
//                        YaRN's are built on the host: the kernels take the table and the factor).  Only the first `rot_dims` dimensions
//                        of a head are rotated.
//   Retention            per head S_t = decay S_(t-1) + k_t v_t^T, o_t = S_t^T q_t (no softmax, no denominator), then o / rms(o) per head
//                        and an output gate silu(g).  State [slot][head][dim][vdim] fp32, carried between steps.  Two options make
//                        it the linear ("lightning") attention of other designs: in_act = 1 applies silu to q, k and v as they
//                        are read, and finish = LP_RET_FINISH_RAW stores o itself (the norm over all heads and the gate follow
//                        in lp_rmsnorm_gated_f32).
//       prefill          chunks of 32 tokens, three kernels: (1) every chunk's own contribution sum_j decay^(len-1-j) k_j v_j^T in
//                        parallel, (2) a scan over the chunks of a request that turns them into the state at each chunk's start and
//                        stores the final state, (3) every chunk's outputs in parallel: decay^(i+1) q_i^T S_start plus the causal
//                        in-chunk part.  Any start position: the scan starts from the stored state when the request has history.
//       decode           one kernel: rotate, update the state in place, read out, normalise, gate.
//   Latent attention     keys and values are up-projections of one cached latent row c (plus one rotated key part shared by all heads).
//                        The kernels work on the cache directly (absorbed form): score = (W_uk^T q_unrot) . c + q_rot . k_rot, output =
//                        W_uv (sum_j p_j c_j); the two per-head products run as batched lp_linear calls around lp_latent_attend.
//                        Sliding window: key j is visible to query i when 0 <= i - j < window (window <= 0: all earlier keys).
//                        Cache: pages of `page_size` rows [c | k_rot] fp32, one page table row per request.
//       lp_latent_prep   RMS-norms the latent (vector gain), rotates the shared key part and writes both to the request's pages;
//                        rotates the query's rotated part in place.
//       lp_latent_attend one CTA per (row, head), its warps split the visible keys: online softmax in fp32, merged at the end.
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

constexpr int RET_CHUNK = LP_RETENTION_CHUNK;
constexpr int RET_CHUNK_THREADS = 256;      // CTA size of the two chunk kernels (their loops stride by blockDim)

// element d of one head's vector x at position pos: rotated when d < rot_dims, copied otherwise
__device__ __forceinline__ float rot_elem(const float* __restrict__ x, int d, int rot_dims, int layout, const float* __restrict__ inv_freq,
                                          float mscale, int pos) {
  if (d >= rot_dims) return x[d];
  const int half = rot_dims >> 1;
  int i, partner;
  bool first;
  if (layout == LP_ROT_INTERLEAVED) {
    i = d >> 1;
    first = (d & 1) == 0;
    partner = first ? d + 1 : d - 1;
  } else {
    first = d < half;
    i = first ? d : d - half;
    partner = first ? d + half : d - half;
  }
  const float ang = (float)pos * inv_freq[i];
  float s, c;
  sincosf(ang, &s, &c);
  s *= mscale;
  c *= mscale;
  // pair (u, v) -> (u c - v s, v c + u s)
  return first ? x[d] * c - x[partner] * s : x[d] * c + x[partner] * s;
}

struct RetArgs {
  const float* qkvg; long long ld; int q_off, k_off, v_off, g_off;
  int heads, dim, vdim;
  const float* decay;
  const float* inv_freq; int rot_dims, rot_layout; float rot_mscale;
  float k_scale, eps;
  float* state; long long slot_stride;
  void* out; long long ldo; int out_fp32;
  int in_act, finish;
};

__device__ __forceinline__ float ret_silu(float z) { return z / (1.0f + expf(-z)); }
// element d of one head's q or k: activation (when asked for), then rotation
__device__ __forceinline__ float ret_qk(const RetArgs& a, const float* __restrict__ x, int d, int pos) {
  if (a.in_act) return ret_silu(x[d]);      // the host admits an activation only without rotation
  return rot_elem(x, d, a.rot_dims, a.rot_layout, a.inv_freq, a.rot_mscale, pos);
}
__device__ __forceinline__ float ret_v(const RetArgs& a, float v) { return a.in_act ? ret_silu(v) : v; }

// (1) U[chunk][head] = sum_j decay^(len-1-j) k_j v_j^T.  4 x 4 outputs per thread; a thread's four columns are vdim/4 apart, so that
// the threads of a warp read consecutive shared-memory words.
__global__ void __launch_bounds__(RET_CHUNK_THREADS)
retention_chunk_state_kernel(RetArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len,
                             const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, float* __restrict__ ws) {
  extern __shared__ float dyn_smem[];
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int s = chunk_seq[c], row0 = chunk_row0[c], len = chunk_len[c];
  const int pos0 = seq_pos0[s] + (row0 - seq_row0[s]);
  const int dimp = ((a.dim + 3) & ~3) + 1, vdimp = (a.vdim + 3) & ~3;      // padded rows: whole 4-tiles, odd stride for k
  float* kd = dyn_smem;                   // [RET_CHUNK][dimp]
  float* vv = kd + RET_CHUNK * dimp;      // [RET_CHUNK][vdimp]
  const float dec = a.decay[h];
  for (int i = tid; i < len * dimp; i += blockDim.x) {
    const int j = i / dimp, d = i % dimp;
    float v = 0.f;
    if (d < a.dim) {
      const float* kr = a.qkvg + (long long)(row0 + j) * a.ld + a.k_off + h * a.dim;
      v = ret_qk(a, kr, d, pos0 + j) * a.k_scale * powf(dec, (float)(len - 1 - j));
    }
    kd[i] = v;
  }
  for (int i = tid; i < len * vdimp; i += blockDim.x) {
    const int j = i / vdimp, d = i % vdimp;
    vv[i] = d < a.vdim ? ret_v(a, a.qkvg[(long long)(row0 + j) * a.ld + a.v_off + h * a.vdim + d]) : 0.f;
  }
  __syncthreads();
  float* U = ws + ((long long)c * a.heads + h) * a.dim * a.vdim;
  const int tiles_y = vdimp >> 2, tiles_x = (a.dim + 3) >> 2;
  for (int tile = tid; tile < tiles_x * tiles_y; tile += blockDim.x) {
    const int x0 = (tile / tiles_y) * 4, ty = tile % tiles_y;
    float acc[4][4];
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[p][q] = 0.f;
    for (int j = 0; j < len; ++j) {
      float k4[4], v4[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        k4[p] = kd[j * dimp + x0 + p];
        v4[p] = vv[j * vdimp + ty + p * tiles_y];
      }
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(k4[p], v4[q], acc[p][q]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int x = x0 + p, y = ty + q * tiles_y;
        if (x < a.dim && y < a.vdim) U[x * a.vdim + y] = acc[p][q];
      }
  }
}

// (2) one thread per state element of a (request, head): ws[chunk] <- state at the chunk's start; the state after the last chunk goes
// to the slot.  The chunks' own contributions are loaded eight at a time (independent loads) ahead of the dependent multiply-adds.
constexpr int SCAN_THREADS = 256, SCAN_BATCH = 8;
__global__ void __launch_bounds__(SCAN_THREADS)
retention_scan_kernel(RetArgs a, const int* __restrict__ seq_chunk0, const int* __restrict__ chunk_len, const int* __restrict__ seq_pos0,
                      const int* __restrict__ seq_slot, float* __restrict__ ws) {
  const int s = blockIdx.x, h = blockIdx.y;
  const long long hs = (long long)a.dim * a.vdim;
  const long long i = (long long)blockIdx.z * SCAN_THREADS + threadIdx.x;
  if (i >= hs) return;
  const int c0 = seq_chunk0[s], c1 = seq_chunk0[s + 1];
  const float dec = a.decay[h];
  const float dec_full = powf(dec, (float)RET_CHUNK);
  float* st = a.state + (long long)seq_slot[s] * a.slot_stride + h * hs + i;
  float S = seq_pos0[s] == 0 ? 0.f : *st;
  const long long stride = (long long)a.heads * hs;
  float* u = ws + ((long long)c0 * a.heads + h) * hs + i;
  for (int c = c0; c < c1; c += SCAN_BATCH) {
    float own[SCAN_BATCH];
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) own[k] = c + k < c1 ? u[k * stride] : 0.f;
#pragma unroll
    for (int k = 0; k < SCAN_BATCH; ++k) {
      if (c + k < c1) {
        const int len = chunk_len[c + k];
        u[k * stride] = S;
        S = fmaf(len == RET_CHUNK ? dec_full : powf(dec, (float)len), S, own[k]);
      }
    }
    u += SCAN_BATCH * stride;
  }
  *st = S;
}

// (3) o_i = decay^(i+1) q_i^T S_start + sum_(j<=i) decay^(i-j) (q_i . k_j) v_j; then o / rms(o) * silu(g).  The chunk's start state is
// staged in shared memory (stage_s; read from global when a head is too large for that); 4 x 4 outputs per thread.
__global__ void __launch_bounds__(RET_CHUNK_THREADS)
retention_chunk_out_kernel(RetArgs a, const int* __restrict__ chunk_seq, const int* __restrict__ chunk_row0, const int* __restrict__ chunk_len,
                           const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, const float* __restrict__ ws, int stage_s) {
  extern __shared__ float dyn_smem[];
  const int c = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int s = chunk_seq[c], row0 = chunk_row0[c], len = chunk_len[c];
  const int pos0 = seq_pos0[s] + (row0 - seq_row0[s]);
  const int dimp = ((a.dim + 3) & ~3) + 1, vdimp = (a.vdim + 3) & ~3;
  float* qs = dyn_smem;                        // [RET_CHUNK][dimp]
  float* ks = qs + RET_CHUNK * dimp;           // [RET_CHUNK][dimp]
  float* vv = ks + RET_CHUNK * dimp;           // [RET_CHUNK][vdimp]
  float* os = vv + RET_CHUNK * vdimp;          // [RET_CHUNK][vdimp]
  float* pp = os + RET_CHUNK * vdimp;          // [RET_CHUNK][RET_CHUNK + 1]
  float* rr = pp + RET_CHUNK * (RET_CHUNK + 1);   // [RET_CHUNK]
  float* Ss = rr + RET_CHUNK;                  // [dim][vdimp] when stage_s
  const float dec = a.decay[h];
  for (int i = tid; i < RET_CHUNK * dimp; i += blockDim.x) {
    const int j = i / dimp, d = i % dimp;
    float qv = 0.f, kv = 0.f;
    if (j < len && d < a.dim) {
      const float* base = a.qkvg + (long long)(row0 + j) * a.ld + h * a.dim;
      qv = ret_qk(a, base + a.q_off, d, pos0 + j);
      kv = ret_qk(a, base + a.k_off, d, pos0 + j) * a.k_scale;
    }
    qs[i] = qv;
    ks[i] = kv;
  }
  for (int i = tid; i < RET_CHUNK * vdimp; i += blockDim.x) {
    const int j = i / vdimp, d = i % vdimp;
    vv[i] = (j < len && d < a.vdim) ? ret_v(a, a.qkvg[(long long)(row0 + j) * a.ld + a.v_off + h * a.vdim + d]) : 0.f;
  }
  const float* S = ws + ((long long)c * a.heads + h) * a.dim * a.vdim;
  if (stage_s)
    for (int i = tid; i < a.dim * vdimp; i += blockDim.x) {
      const int d = i / vdimp, y = i % vdimp;
      Ss[i] = y < a.vdim ? S[d * a.vdim + y] : 0.f;
    }
  __syncthreads();
  // in-chunk scores, 4 x 4 per thread (rows i0 .. i0+3, columns tj, tj+8, tj+16, tj+24)
  for (int tile = tid; tile < (RET_CHUNK / 4) * (RET_CHUNK / 4); tile += blockDim.x) {
    const int i0 = (tile / (RET_CHUNK / 4)) * 4, tj = tile % (RET_CHUNK / 4);
    float acc[4][4];
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[p][q] = 0.f;
    for (int d = 0; d < a.dim; ++d) {
      float q4[4], k4[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        q4[p] = qs[(i0 + p) * dimp + d];
        k4[p] = ks[(tj + p * (RET_CHUNK / 4)) * dimp + d];
      }
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(q4[p], k4[q], acc[p][q]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const int i = i0 + p, j = tj + q * (RET_CHUNK / 4);
        pp[i * (RET_CHUNK + 1) + j] = (j <= i && i < len) ? acc[p][q] * powf(dec, (float)(i - j)) : 0.f;
      }
  }
  __syncthreads();
  const int tiles_y = vdimp >> 2, tiles_i = (len + 3) >> 2;
  for (int tile = tid; tile < tiles_i * tiles_y; tile += blockDim.x) {
    const int i0 = (tile / tiles_y) * 4, ty = tile % tiles_y;
    float acc[4][4];
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[p][q] = 0.f;
    for (int d = 0; d < a.dim; ++d) {
      float q4[4], s4[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        q4[p] = qs[(i0 + p) * dimp + d];
        const int y = ty + p * tiles_y;
        s4[p] = stage_s ? Ss[d * vdimp + y] : (y < a.vdim ? S[d * a.vdim + y] : 0.f);
      }
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(q4[p], s4[q], acc[p][q]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p) {
      const float sc = powf(dec, (float)(i0 + p + 1));
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[p][q] *= sc;
    }
    const int jmax = min(i0 + 3, len - 1);
    for (int j = 0; j <= jmax; ++j) {
      float p4[4], v4[4];
#pragma unroll
      for (int p = 0; p < 4; ++p) {
        p4[p] = pp[(i0 + p) * (RET_CHUNK + 1) + j];
        v4[p] = vv[j * vdimp + ty + p * tiles_y];
      }
#pragma unroll
      for (int p = 0; p < 4; ++p)
#pragma unroll
        for (int q = 0; q < 4; ++q) acc[p][q] = fmaf(p4[p], v4[q], acc[p][q]);
    }
#pragma unroll
    for (int p = 0; p < 4; ++p)
#pragma unroll
      for (int q = 0; q < 4; ++q) os[(i0 + p) * vdimp + ty + q * tiles_y] = acc[p][q];
  }
  __syncthreads();
  if (a.finish == LP_RET_FINISH_RAW) {      // o itself: what follows it is another kernel's
    for (int e = tid; e < len * a.vdim; e += blockDim.x) {
      const int i = e / a.vdim, y = e % a.vdim;
      const long long o = (long long)(row0 + i) * a.ldo + h * a.vdim + y;
      if (a.out_fp32) reinterpret_cast<float*>(a.out)[o] = os[i * vdimp + y];
      else reinterpret_cast<bf16*>(a.out)[o] = __float2bfloat16(os[i * vdimp + y]);
    }
    return;
  }
  // one warp per row: root mean square over the head's vdim outputs
  const int warp = tid >> 5, lane = tid & 31, nwarp = blockDim.x >> 5;
  for (int i = warp; i < len; i += nwarp) {
    float ss = 0.f;
    for (int y = lane; y < a.vdim; y += 32) ss = fmaf(os[i * vdimp + y], os[i * vdimp + y], ss);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
    if (lane == 0) rr[i] = 1.0f / sqrtf(ss / (float)a.vdim + a.eps);
  }
  __syncthreads();
  for (int e = tid; e < len * a.vdim; e += blockDim.x) {
    const int i = e / a.vdim, y = e % a.vdim;
    const float g = a.qkvg[(long long)(row0 + i) * a.ld + a.g_off + h * a.vdim + y];
    const float v = os[i * vdimp + y] * rr[i] * (g / (1.0f + expf(-g)));
    const long long o = (long long)(row0 + i) * a.ldo + h * a.vdim + y;
    if (a.out_fp32) reinterpret_cast<float*>(a.out)[o] = v;
    else reinterpret_cast<bf16*>(a.out)[o] = __float2bfloat16(v);
  }
}

// decode: one new row per request.  Threads own state columns; with vdim < blockDim several thread groups split the dim rows.
constexpr int RET_DEC_THREADS = 256;
__global__ void __launch_bounds__(RET_DEC_THREADS)
retention_decode_kernel(RetArgs a, const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot) {
  extern __shared__ float dyn_smem[];
  const int s = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
  const int row = seq_row0[s], pos = seq_pos0[s];
  float* qs = dyn_smem;            // [dim]
  float* ks = qs + a.dim;          // [dim]
  float* vv = ks + a.dim;          // [vdim]
  float* os = vv + a.vdim;         // [vdim]
  float* part = os + a.vdim;       // [groups][vdim]
  __shared__ float red[RET_DEC_THREADS / 32];
  const float* base = a.qkvg + (long long)row * a.ld;
  for (int d = tid; d < a.dim; d += blockDim.x) {
    qs[d] = ret_qk(a, base + a.q_off + h * a.dim, d, pos);
    ks[d] = ret_qk(a, base + a.k_off + h * a.dim, d, pos) * a.k_scale;
  }
  for (int y = tid; y < a.vdim; y += blockDim.x) vv[y] = ret_v(a, base[a.v_off + h * a.vdim + y]);
  __syncthreads();
  const float dec = a.decay[h];
  const bool fresh = pos == 0;
  float* st = a.state + (long long)seq_slot[s] * a.slot_stride + (long long)h * a.dim * a.vdim;
  const int groups = a.vdim >= (int)blockDim.x ? 1 : (int)blockDim.x / a.vdim;
  const int g = tid / a.vdim;
  const int per = (a.dim + groups - 1) / groups;
  if (g < groups) {
    const int d0 = g * per, d1 = min(a.dim, d0 + per);
    for (int y = tid % a.vdim; y < a.vdim; y += blockDim.x) {
      float acc = 0.f;
#pragma unroll 8
      for (int d = d0; d < d1; ++d) {
        const float old = fresh ? 0.f : st[(long long)d * a.vdim + y];
        const float S = fmaf(dec, old, ks[d] * vv[y]);
        st[(long long)d * a.vdim + y] = S;
        acc = fmaf(S, qs[d], acc);
      }
      part[g * a.vdim + y] = acc;
    }
  }
  __syncthreads();
  float ss = 0.f;
  for (int y = tid; y < a.vdim; y += blockDim.x) {
    float acc = 0.f;
    for (int gg = 0; gg < groups; ++gg) acc += part[gg * a.vdim + y];
    os[y] = acc;
    ss = fmaf(acc, acc, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  float tot = 0.f;
  for (int w = 0; w < RET_DEC_THREADS / 32; ++w) tot += red[w];
  const float r = 1.0f / sqrtf(tot / (float)a.vdim + a.eps);
  for (int y = tid; y < a.vdim; y += blockDim.x) {
    float v = os[y];
    if (a.finish != LP_RET_FINISH_RAW) {
      const float gt = base[a.g_off + h * a.vdim + y];
      v = v * r * (gt / (1.0f + expf(-gt)));
    }
    const long long o = (long long)row * a.ldo + h * a.vdim + y;
    if (a.out_fp32) reinterpret_cast<float*>(a.out)[o] = v;
    else reinterpret_cast<bf16*>(a.out)[o] = __float2bfloat16(v);
  }
}

// ---------------------------------------------------------------------------------------------------------------------------------
// latent attention
// ---------------------------------------------------------------------------------------------------------------------------------
struct LatArgs {
  float* q; long long ldq;
  const float* dkv; long long lddkv;
  int heads, dim, rot_dim, kv_rank;
  const float* c_gain; float eps;
  const float* inv_freq; int rot_dims, rot_layout; float rot_mscale;
  float* cache; int page_size;
  const int* page_table; int max_pages;
  int window; float scale;
  const float* sink;                      // [heads] or null: exp(sink_h) joins the softmax denominator (no key, no value, not scaled)
  const float* gate; long long ldg;       // [rows, ldg] or null: head h's output is multiplied by sigmoid(gate[r, h])
};

__device__ __forceinline__ float lat_gate(const LatArgs& a, int r, int h) {
  return a.gate != nullptr ? 1.0f / (1.0f + expf(-a.gate[(long long)r * a.ldg + h])) : 1.0f;
}

__device__ __forceinline__ float* lat_cache_row(const LatArgs& a, int seq, int pos) {
  const int page = a.page_table[(long long)seq * a.max_pages + pos / a.page_size];
  return a.cache + ((long long)page * a.page_size + pos % a.page_size) * (a.kv_rank + a.rot_dim);
}

__global__ void __launch_bounds__(128)
latent_prep_kernel(LatArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos) {
  __shared__ float red[4];
  const int r = blockIdx.x, tid = threadIdx.x;
  if (r >= R) return;
  const int pos = row_pos[r];
  const float* src = a.dkv + (long long)r * a.lddkv;
  float ss = 0.f;
  for (int c = tid; c < a.kv_rank; c += blockDim.x) ss = fmaf(src[c], src[c], ss);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  if ((tid & 31) == 0) red[tid >> 5] = ss;
  __syncthreads();
  const float inv = 1.0f / sqrtf((red[0] + red[1] + red[2] + red[3]) / (float)a.kv_rank + a.eps);
  float* dst = lat_cache_row(a, row_seq[r], pos);
  for (int c = tid; c < a.kv_rank; c += blockDim.x) dst[c] = src[c] * inv * a.c_gain[c];
  for (int d = tid; d < a.rot_dim; d += blockDim.x)
    dst[a.kv_rank + d] = rot_elem(src + a.kv_rank, d, a.rot_dims, a.rot_layout, a.inv_freq, a.rot_mscale, pos);
  // the rotated part of every head's query, in place: one thread per pair reads both members, then writes both
  float* q = a.q + (long long)r * a.ldq;
  const int per = a.dim + a.rot_dim, half = a.rot_dims >> 1;
  for (int p = tid; p < a.heads * half; p += blockDim.x) {
    float* x = q + (p / half) * per + a.dim;
    const int i = p % half;
    const int d0 = a.rot_layout == LP_ROT_INTERLEAVED ? 2 * i : i;
    const int d1 = a.rot_layout == LP_ROT_INTERLEAVED ? 2 * i + 1 : i + half;
    const float u = rot_elem(x, d0, a.rot_dims, a.rot_layout, a.inv_freq, a.rot_mscale, pos);
    const float v = rot_elem(x, d1, a.rot_dims, a.rot_layout, a.inv_freq, a.rot_mscale, pos);
    x[d0] = u;
    x[d1] = v;
  }
}

// One CTA per (row, head): its warps take every LAT_WARPS-th visible key with an online softmax of their own, then the partial
// (maximum, denominator, weighted sum) triples are merged.  NR = ceil(kv_rank / 32) accumulators per lane.
constexpr int LAT_WARPS = 16;
constexpr int LAT_SPLIT_MAX_RANK = 512;      // larger latents take the per-row kernel
constexpr int LAT_MAX_RANK = 1024;
template <int NR>
__global__ void __launch_bounds__(LAT_WARPS * 32)
latent_attend_kernel(LatArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos, const float* __restrict__ q_abs,
                     long long ldqa, void* __restrict__ out, long long ldo, int out_fp32) {
  __shared__ float s_acc[LAT_WARPS][LAT_SPLIT_MAX_RANK];
  __shared__ float s_mx[LAT_WARPS], s_den[LAT_WARPS];
  const int item = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item >= R * a.heads) return;
  const int r = item / a.heads, h = item % a.heads;
  const int seq = row_seq[r], pos = row_pos[r];
  const float* qa = q_abs + (long long)r * ldqa + (long long)h * a.kv_rank;
  const float* qr = a.q + (long long)r * a.ldq + (long long)h * (a.dim + a.rot_dim) + a.dim;
  float qv[NR], qrv[NR], acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int c = lane + 32 * i;
    qv[i] = c < a.kv_rank ? qa[c] : 0.f;
    qrv[i] = c < a.rot_dim ? qr[c] : 0.f;      // rot_dim <= 32 * NR (checked by the host): lanes hold it strided as well
    acc[i] = 0.f;
  }
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  // the sink is a key without a value whose score is sink_h as it stands: warp 0 starts from it
  const bool sunk = a.sink != nullptr && warp == 0;
  float mx = sunk ? a.sink[h] : -INFINITY, den = sunk ? 1.f : 0.f;
  // two keys per turn: their score reductions overlap, one rescale of the running sums serves both
  for (int j = lo + warp; j <= pos; j += 2 * LAT_WARPS) {
    const bool two = j + LAT_WARPS <= pos;
    const float* kv0 = lat_cache_row(a, seq, j);
    const float* kv1 = two ? lat_cache_row(a, seq, j + LAT_WARPS) : kv0;
    float cv0[NR], cv1[NR];
    float sc0 = 0.f, sc1 = 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int c = lane + 32 * i;
      cv0[i] = c < a.kv_rank ? kv0[c] : 0.f;
      cv1[i] = c < a.kv_rank ? kv1[c] : 0.f;
      sc0 = fmaf(qv[i], cv0[i], sc0);
      sc1 = fmaf(qv[i], cv1[i], sc1);
      if (c < a.rot_dim) {
        sc0 = fmaf(qrv[i], kv0[a.kv_rank + c], sc0);
        sc1 = fmaf(qrv[i], kv1[a.kv_rank + c], sc1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sc0 += __shfl_xor_sync(0xffffffffu, sc0, o);
      sc1 += __shfl_xor_sync(0xffffffffu, sc1, o);
    }
    sc0 *= a.scale;
    sc1 = two ? sc1 * a.scale : -INFINITY;
    const float mn = fmaxf(mx, fmaxf(sc0, sc1));
    const float corr = expf(mx - mn);      // exp(-inf) = 0 on the first turn
    const float p0 = expf(sc0 - mn), p1 = expf(sc1 - mn);
    den = den * corr + p0 + p1;
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] = fmaf(p1, cv1[i], fmaf(p0, cv0[i], acc[i] * corr));
    mx = mn;
  }
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int c = lane + 32 * i;
    if (c < a.kv_rank) s_acc[warp][c] = acc[i];
  }
  if (lane == 0) {
    s_mx[warp] = mx;
    s_den[warp] = den;
  }
  __syncthreads();
  float top = s_mx[0];
#pragma unroll
  for (int w = 1; w < LAT_WARPS; ++w) top = fmaxf(top, s_mx[w]);
  float f[LAT_WARPS], total = 0.f;
#pragma unroll
  for (int w = 0; w < LAT_WARPS; ++w) {
    f[w] = s_den[w] > 0.f ? expf(s_mx[w] - top) : 0.f;      // a warp without keys contributes nothing
    total = fmaf(s_den[w], f[w], total);
  }
  const float inv = lat_gate(a, r, h) / total;
  for (int c = threadIdx.x; c < a.kv_rank; c += blockDim.x) {
    float v = 0.f;
#pragma unroll
    for (int w = 0; w < LAT_WARPS; ++w) v = fmaf(s_acc[w][c], f[w], v);
    const long long o = (long long)r * ldo + (long long)h * a.kv_rank + c;
    if (out_fp32) reinterpret_cast<float*>(out)[o] = v * inv;
    else reinterpret_cast<bf16*>(out)[o] = __float2bfloat16(v * inv);
  }
}

// Many rows (prompts): one CTA per row and group of LAT_ROW_HEADS heads, one warp per head, every warp walks all visible keys.
// The heads of a row read the same cache rows at about the same time, so the cache traffic of a row is paid once per CTA (L1), and
// neighbouring rows overlap in all but one key (L2).
constexpr int LAT_ROW_HEADS = 4;
template <int NR>
__global__ void __launch_bounds__(LAT_ROW_HEADS * 32)
latent_attend_rows_kernel(LatArgs a, int R, const int* __restrict__ row_seq, const int* __restrict__ row_pos, const float* __restrict__ q_abs,
                          long long ldqa, void* __restrict__ out, long long ldo, int out_fp32) {
  const int r = blockIdx.x;
  const int h = blockIdx.y * LAT_ROW_HEADS + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (r >= R || h >= a.heads) return;
  const int seq = row_seq[r], pos = row_pos[r];
  const float* qa = q_abs + (long long)r * ldqa + (long long)h * a.kv_rank;
  const float* qr = a.q + (long long)r * a.ldq + (long long)h * (a.dim + a.rot_dim) + a.dim;
  float qv[NR], qrv[NR], acc[NR];
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int c = lane + 32 * i;
    qv[i] = c < a.kv_rank ? qa[c] : 0.f;
    qrv[i] = c < a.rot_dim ? qr[c] : 0.f;
    acc[i] = 0.f;
  }
  const int lo = (a.window > 0 && pos - a.window + 1 > 0) ? pos - a.window + 1 : 0;
  float mx = a.sink != nullptr ? a.sink[h] : -INFINITY, den = a.sink != nullptr ? 1.f : 0.f;
  // two keys per turn: their score reductions overlap, one rescale of the running sums serves both
  for (int j = lo; j <= pos; j += 2 * 1) {
    const bool two = j + 1 <= pos;
    const float* kv0 = lat_cache_row(a, seq, j);
    const float* kv1 = two ? lat_cache_row(a, seq, j + 1) : kv0;
    float cv0[NR], cv1[NR];
    float sc0 = 0.f, sc1 = 0.f;
#pragma unroll
    for (int i = 0; i < NR; ++i) {
      const int c = lane + 32 * i;
      cv0[i] = c < a.kv_rank ? kv0[c] : 0.f;
      cv1[i] = c < a.kv_rank ? kv1[c] : 0.f;
      sc0 = fmaf(qv[i], cv0[i], sc0);
      sc1 = fmaf(qv[i], cv1[i], sc1);
      if (c < a.rot_dim) {
        sc0 = fmaf(qrv[i], kv0[a.kv_rank + c], sc0);
        sc1 = fmaf(qrv[i], kv1[a.kv_rank + c], sc1);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      sc0 += __shfl_xor_sync(0xffffffffu, sc0, o);
      sc1 += __shfl_xor_sync(0xffffffffu, sc1, o);
    }
    sc0 *= a.scale;
    sc1 = two ? sc1 * a.scale : -INFINITY;
    const float mn = fmaxf(mx, fmaxf(sc0, sc1));
    const float corr = expf(mx - mn);      // exp(-inf) = 0 on the first turn
    const float p0 = expf(sc0 - mn), p1 = expf(sc1 - mn);
    den = den * corr + p0 + p1;
#pragma unroll
    for (int i = 0; i < NR; ++i) acc[i] = fmaf(p1, cv1[i], fmaf(p0, cv0[i], acc[i] * corr));
    mx = mn;
  }
  const float inv = lat_gate(a, r, h) / den;
#pragma unroll
  for (int i = 0; i < NR; ++i) {
    const int c = lane + 32 * i;
    if (c < a.kv_rank) {
      const long long o = (long long)r * ldo + (long long)h * a.kv_rank + c;
      if (out_fp32) reinterpret_cast<float*>(out)[o] = acc[i] * inv;
      else reinterpret_cast<bf16*>(out)[o] = __float2bfloat16(acc[i] * inv);
    }
  }
}

// raise a kernel's dynamic shared-memory limit only when a launch needs more than any launch before it (no runtime call on the
// steady path, so the steady path can be captured into a CUDA graph)
template <typename K>
static cudaError_t ensure_smem(K kern, size_t bytes, size_t& have) {
  if (bytes <= have) return cudaSuccess;
  const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
  if (e == cudaSuccess) have = bytes;
  return e;
}
static size_t g_smem_chunk_state = 48 * 1024, g_smem_chunk_out = 48 * 1024, g_smem_ret_decode = 48 * 1024;

static int fill_ret(RetArgs& a, const lp_retention_desc* d) {
  LP_REQUIRE(d != nullptr && d->qkvg != nullptr && d->decay != nullptr && d->state != nullptr && d->out != nullptr,
             "lp_retention: null operand");
  LP_REQUIRE(d->heads > 0 && d->dim > 0 && d->vdim > 0, "lp_retention: bad sizes heads=%d dim=%d vdim=%d", d->heads, d->dim, d->vdim);
  LP_REQUIRE(d->rot_dims >= 0 && d->rot_dims <= d->dim && d->rot_dims % 2 == 0, "lp_retention: rot_dims=%d must be even and <= dim=%d",
             d->rot_dims, d->dim);
  LP_REQUIRE(d->rot_dims == 0 || d->inv_freq != nullptr, "lp_retention: rotation without a frequency table");
  a.qkvg = d->qkvg; a.ld = d->ld; a.q_off = d->q_off; a.k_off = d->k_off; a.v_off = d->v_off; a.g_off = d->g_off;
  a.heads = d->heads; a.dim = d->dim; a.vdim = d->vdim;
  a.decay = d->decay;
  a.inv_freq = d->inv_freq; a.rot_dims = d->rot_dims; a.rot_layout = d->rot_layout; a.rot_mscale = d->rot_mscale;
  a.k_scale = d->k_scale; a.eps = d->eps;
  a.in_act = d->in_act; a.finish = d->finish;
  LP_REQUIRE(d->in_act == 0 || d->rot_dims == 0, "lp_retention: an input activation together with rotation is not supported");
  LP_REQUIRE(d->finish == LP_RET_FINISH_GATED_NORM || d->finish == LP_RET_FINISH_RAW, "lp_retention: bad finish %d", d->finish);
  a.state = d->state; a.slot_stride = d->slot_stride;
  a.out = d->out; a.ldo = d->ldo; a.out_fp32 = d->out_fp32;
  return 0;
}

static int fill_lat(LatArgs& a, const lp_latent_desc* d) {
  LP_REQUIRE(d != nullptr && d->q != nullptr && d->cache != nullptr && d->page_table != nullptr, "lp_latent: null operand");
  LP_REQUIRE(d->heads > 0 && d->dim >= 0 && d->rot_dim >= 0 && d->kv_rank > 0 && d->page_size > 0 && d->max_pages > 0,
             "lp_latent: bad sizes");
  LP_REQUIRE(d->rot_dims >= 0 && d->rot_dims <= d->rot_dim && d->rot_dims % 2 == 0, "lp_latent: rot_dims=%d must be even and <= rot_dim=%d",
             d->rot_dims, d->rot_dim);
  LP_REQUIRE(d->rot_dims == 0 || d->inv_freq != nullptr, "lp_latent: rotation without a frequency table");
  a.q = d->q; a.ldq = d->ldq; a.dkv = d->dkv; a.lddkv = d->lddkv;
  a.heads = d->heads; a.dim = d->dim; a.rot_dim = d->rot_dim; a.kv_rank = d->kv_rank;
  a.c_gain = d->c_gain; a.eps = d->eps;
  a.inv_freq = d->inv_freq; a.rot_dims = d->rot_dims; a.rot_layout = d->rot_layout; a.rot_mscale = d->rot_mscale;
  a.cache = d->cache; a.page_size = d->page_size; a.page_table = d->page_table; a.max_pages = d->max_pages;
  a.window = d->window; a.scale = d->scale;
  a.sink = d->sink; a.gate = d->gate; a.ldg = d->ldg;
  return 0;
}

}  // namespace lp

using namespace lp;

extern "C" size_t lp_retention_workspace_bytes(int n_chunks, int heads, int dim, int vdim) {
  return (size_t)n_chunks * heads * dim * vdim * sizeof(float);
}

extern "C" int lp_retention_prefill(const lp_retention_desc* d, int n_seqs, int n_chunks, const int* seq_row0, const int* seq_pos0,
                                    const int* seq_slot, const int* seq_chunk0, const int* chunk_seq, const int* chunk_row0,
                                    const int* chunk_len, void* ws, size_t ws_bytes, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  RetArgs a;
  if (int rc = fill_ret(a, d)) return rc;
  LP_REQUIRE(n_seqs >= 0 && n_chunks >= 0, "lp_retention_prefill: bad counts");
  if (n_seqs == 0 || n_chunks == 0) return 0;
  LP_REQUIRE(ws != nullptr && ws_bytes >= lp_retention_workspace_bytes(n_chunks, d->heads, d->dim, d->vdim),
             "lp_retention_prefill: workspace too small");
  float* w = reinterpret_cast<float*>(ws);
  const size_t dimp = ((d->dim + 3) & ~3) + 1, vdimp = (d->vdim + 3) & ~3;
  const size_t smem1 = (size_t)RET_CHUNK * (dimp + vdimp) * sizeof(float);
  size_t smem3 = ((size_t)RET_CHUNK * (2 * dimp + 2 * vdimp) + RET_CHUNK * (RET_CHUNK + 1) + RET_CHUNK) * sizeof(float);
  LP_REQUIRE(smem3 <= 200 * 1024, "lp_retention_prefill: dim=%d vdim=%d do not fit the chunk kernel's shared memory", d->dim, d->vdim);
  const int stage_s = smem3 + (size_t)d->dim * vdimp * sizeof(float) <= 200 * 1024;      // the chunk's start state next to the operands
  if (stage_s) smem3 += (size_t)d->dim * vdimp * sizeof(float);
  LP_CHECK_CUDA(ensure_smem(retention_chunk_state_kernel, smem1, g_smem_chunk_state));
  LP_CHECK_CUDA(ensure_smem(retention_chunk_out_kernel, smem3, g_smem_chunk_out));
  retention_chunk_state_kernel<<<dim3(n_chunks, d->heads), RET_CHUNK_THREADS, smem1, stream>>>(a, chunk_seq, chunk_row0, chunk_len, seq_row0, seq_pos0, w);
  LP_CHECK_CUDA(cudaGetLastError());
  retention_scan_kernel<<<dim3(n_seqs, d->heads, (d->dim * d->vdim + SCAN_THREADS - 1) / SCAN_THREADS), SCAN_THREADS, 0, stream>>>(
      a, seq_chunk0, chunk_len, seq_pos0, seq_slot, w);
  LP_CHECK_CUDA(cudaGetLastError());
  retention_chunk_out_kernel<<<dim3(n_chunks, d->heads), RET_CHUNK_THREADS, smem3, stream>>>(a, chunk_seq, chunk_row0, chunk_len, seq_row0, seq_pos0, w,
                                                                                stage_s);
  LP_CHECK_CUDA(cudaGetLastError());
  note_launch(3);
  return 0;
}

extern "C" int lp_retention_decode(const lp_retention_desc* d, int n_seqs, const int* seq_row0, const int* seq_pos0, const int* seq_slot,
                                   void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  RetArgs a;
  if (int rc = fill_ret(a, d)) return rc;
  if (n_seqs <= 0) return 0;
  const int groups = d->vdim >= RET_DEC_THREADS ? 1 : RET_DEC_THREADS / d->vdim;
  const size_t smem = ((size_t)2 * d->dim + 2 * d->vdim + (size_t)groups * d->vdim) * sizeof(float);
  LP_REQUIRE(smem <= 200 * 1024, "lp_retention_decode: dim=%d vdim=%d do not fit shared memory", d->dim, d->vdim);
  LP_CHECK_CUDA(ensure_smem(retention_decode_kernel, smem, g_smem_ret_decode));
  retention_decode_kernel<<<dim3(n_seqs, d->heads), RET_DEC_THREADS, smem, stream>>>(a, seq_row0, seq_pos0, seq_slot);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_latent_prep(const lp_latent_desc* d, int R, const int* row_seq, const int* row_pos, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LatArgs a;
  if (int rc = fill_lat(a, d)) return rc;
  LP_REQUIRE(d->dkv != nullptr && d->c_gain != nullptr && row_seq != nullptr && row_pos != nullptr, "lp_latent_prep: null operand");
  if (R <= 0) return 0;
  latent_prep_kernel<<<R, 128, 0, stream>>>(a, R, row_seq, row_pos);
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}

extern "C" int lp_latent_attend(const lp_latent_desc* d, int R, const int* row_seq, const int* row_pos, const float* q_abs, long long ldqa,
                                void* out, long long ldo, int out_fp32, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LatArgs a;
  if (int rc = fill_lat(a, d)) return rc;
  LP_REQUIRE(q_abs != nullptr && out != nullptr && row_seq != nullptr && row_pos != nullptr, "lp_latent_attend: null operand");
  LP_REQUIRE(d->kv_rank <= LAT_MAX_RANK && d->rot_dim <= LAT_MAX_RANK, "lp_latent_attend: kv_rank=%d / rot_dim=%d > %d is not instantiated",
             d->kv_rank, d->rot_dim, LAT_MAX_RANK);
  if (R <= 0) return 0;
  const int nr = ((d->kv_rank > d->rot_dim ? d->kv_rank : d->rot_dim) + 31) / 32;      // lanes hold both vectors strided by 32
  if (R > LP_LATENT_SPLIT_ROWS || d->kv_rank > LAT_SPLIT_MAX_RANK) {      // prompts: a CTA per row, a warp per head
    const dim3 grid(R, (d->heads + LAT_ROW_HEADS - 1) / LAT_ROW_HEADS);
    const int threads = (d->heads < LAT_ROW_HEADS ? d->heads : LAT_ROW_HEADS) * 32;
    if (nr <= 2) latent_attend_rows_kernel<2><<<grid, threads, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 4) latent_attend_rows_kernel<4><<<grid, threads, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 8) latent_attend_rows_kernel<8><<<grid, threads, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 16) latent_attend_rows_kernel<16><<<grid, threads, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else latent_attend_rows_kernel<32><<<grid, threads, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
  } else {                             // few rows (decoding): a CTA per (row, head), its warps split the keys
    const unsigned grid = (unsigned)((long long)R * d->heads);
    if (nr <= 2) latent_attend_kernel<2><<<grid, LAT_WARPS * 32, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 4) latent_attend_kernel<4><<<grid, LAT_WARPS * 32, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 8) latent_attend_kernel<8><<<grid, LAT_WARPS * 32, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else if (nr <= 16) latent_attend_kernel<16><<<grid, LAT_WARPS * 32, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
    else latent_attend_kernel<32><<<grid, LAT_WARPS * 32, 0, stream>>>(a, R, row_seq, row_pos, q_abs, ldqa, out, ldo, out_fp32);
  }
  note_launch();
  LP_CHECK_CUDA(cudaGetLastError());
  return 0;
}
