// leopard_b200 — mLSTM: a matrix memory per head with exponential gates and a running stabiliser, everything after the projections
// in 32-bit floats.
//
// Per head, with q (scaled by q_scale), k [dim], v [vdim] and two gate pre-activations a_i, a_f of the token:
//   i = cap * tanh((a_i + b_i) / cap)                       log input gate
//   f = logsigmoid(cap * tanh((a_f + b_f) / cap))           log forget gate
//   m_t = max(f + m_(t-1), i),  m_(-1) = 0                  running maximum (starts at 0, not at minus infinity)
//   S_t = exp(f + m_(t-1) - m_t) S_(t-1) + exp(i - m_t) k v^T        S [dim, vdim], starts at zero
//   n_t = the same recurrence with k alone                            n [dim]
//   o_t = S_t^T q / (max(|n_t . q|, exp(-m_t)) + 1e-6)
// then o / rms(o) per head (eps), times a gain per channel, times sigmoid(g).
//
//   lp_mlstm   three kernels for prompts, portions and one-token steps alike:
//     gates    a CTA per (request, head): the gate transforms and the running maximum of all tokens (a scan, 256 tokens a turn), written
//              as the two factors exp(f + m_(t-1) - m_t), exp(i - m_t) and m_t per (token, head).
//     scan     a CTA per (request, head, tile of 32 state columns); the normaliser n is one more COLUMN of the state (its "value" is
//              1), so S and n share the code.  A thread owns 8 or 16 rows of one column in registers (threadIdx.y picks the rows).  Tokens
//              are staged in shared memory 16 at a time, the next stage travelling from global memory into registers meanwhile;
//              the 16 state updates of a stage run without any synchronisation, and the partial read-outs of the row groups meet in
//              shared memory once per stage.  The state is read from and written to the request's slot ([dim + 1][vdim + 1] per
//              head: S | n, and m in the last row) — a request at position 0 starts from zero without reading it.
//     finish   a warp per (row, head): denominator, unit RMS, gain, gate.
// The recurrence is run token by token in every case, so a row's result does not depend on how the tokens were cut into steps (the
// scan of the maximum regroups max and + only, which are exact up to the rounding of the sums of log gates).
#include "lp_host.h"
#include "../../include/leopard_b200.h"

namespace lp {

typedef __nv_bfloat16 bf16;

struct MlstmArgs {
  const float* proj; long long ld; int q_off, k_off, v_off, g_off, i_off, f_off;
  int heads, dim, vdim;
  const float* i_bias; const float* f_bias;
  float gate_cap, q_scale, eps;
  const float* out_gain;
  float* state; long long slot_stride;
  void* out; long long ldo; int out_fp32;
};

constexpr int MLSTM_COLS = 32;      // state columns per CTA
constexpr int MLSTM_ROWS = 16;      // most state rows per thread
constexpr int MLSTM_TOK = 16;       // tokens staged at a time
constexpr int MLSTM_MAX_GROUPS = 16;      // row groups (threadIdx.y) per CTA: dim <= 256

__device__ __forceinline__ float mlstm_logsigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

// The gates of every token, one CTA per (request, head), 32 tokens a warp and turn.  m_t = max(f_t + m_(t-1), i_t) is a chain of maps
// m -> max(m + a, b); two such maps compose to one of the same kind, (a1, b1) then (a2, b2) = (a1 + a2, max(b1 + a2, b2)), so the 32
// maps of a warp are combined by a butterfly of shuffles into every lane's map "the warp's tokens before mine", the warps' whole maps
// meet in shared memory, and applied in order to the m carried from the turn before they give m_(t-1); m_t follows locally.
// Written per (row, head): exp(f + m_(t-1) - m_t), exp(i - m_t) and m_t.  m lives in the last row of the head's state ([dim][0] of
// [dim + 1][vdim + 1]); only this kernel touches it.
constexpr int MLSTM_GATE_WARPS = 8;
__global__ void __launch_bounds__(MLSTM_GATE_WARPS * 32)
mlstm_gate_kernel(MlstmArgs a, int n_seqs, const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                  float* __restrict__ gates) {
  __shared__ float wa_s[MLSTM_GATE_WARPS], wb_s[MLSTM_GATE_WARPS];
  const int item = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  if (item >= n_seqs * a.heads) return;
  const int s = item / a.heads, h = item % a.heads;
  const int row0 = seq_row0[s], len = seq_row0[s + 1] - row0;
  float* m_slot = a.state + (long long)seq_slot[s] * a.slot_stride + ((long long)h * (a.dim + 1) + a.dim) * (a.vdim + 1);
  float m = seq_pos0[s] > 0 ? *m_slot : 0.f;      // the running maximum starts at 0
  const float bi = a.i_bias[h], bf = a.f_bias[h];
  for (int c0 = 0; c0 < len; c0 += MLSTM_GATE_WARPS * 32) {
    const int t = c0 + warp * 32 + lane;
    float gi = -INFINITY, gf = 0.f;      // a lane past the end is the identity map
    if (t < len) {
      const float* row = a.proj + (long long)(row0 + t) * a.ld;
      gi = a.gate_cap * tanhf((row[a.i_off + h] + bi) / a.gate_cap);
      gf = mlstm_logsigmoid(a.gate_cap * tanhf((row[a.f_off + h] + bf) / a.gate_cap));
    }
    float ta = gf, tb = gi;              // the map of this lane's group of tokens
    float pa = 0.f, pb = -INFINITY;      // the map of the warp's tokens before this lane
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      const float oa = __shfl_xor_sync(0xffffffffu, ta, o), ob = __shfl_xor_sync(0xffffffffu, tb, o);
      if (lane & o) {      // the partner's group comes first
        pb = fmaxf(ob + pa, pb);
        pa = oa + pa;
        tb = fmaxf(ob + ta, tb);
      } else {
        tb = fmaxf(tb + oa, ob);
      }
      ta = ta + oa;
    }
    if (lane == 0) {
      wa_s[warp] = ta;
      wb_s[warp] = tb;
    }
    __syncthreads();
    float m_warp = m;                    // m before this warp's tokens, and after the whole turn
    float m_next = m;
#pragma unroll
    for (int w = 0; w < MLSTM_GATE_WARPS; ++w) {
      m_next = fmaxf(m_next + wa_s[w], wb_s[w]);
      if (w + 1 == warp) m_warp = m_next;
    }
    const float m_before = fmaxf(m_warp + pa, pb);
    const float m_here = fmaxf(gf + m_before, gi);
    if (t < len) {
      float* g = gates + ((long long)(row0 + t) * a.heads + h) * 3;
      g[0] = expf(gf + m_before - m_here);
      g[1] = expf(gi - m_here);
      g[2] = m_here;
    }
    m = m_next;
    __syncthreads();                     // the warps' maps have been read
  }
  if (threadIdx.x == 0) *m_slot = m;
}

// num [rows][heads][vdim + 1] (the last column is n . q); gates [rows][heads][3] from mlstm_gate_kernel
template <int ROWS>      // state rows per thread: 8 (dim <= 128: twice the warps to hide the latencies of a stage) or 16
__global__ void __launch_bounds__(MLSTM_COLS * MLSTM_MAX_GROUPS)
mlstm_scan_kernel(MlstmArgs a, const int* __restrict__ seq_row0, const int* __restrict__ seq_pos0, const int* __restrict__ seq_slot,
                  const float* __restrict__ gates, float* __restrict__ num) {
  extern __shared__ float dyn_smem[];
  constexpr int PF = MLSTM_TOK * ROWS / MLSTM_COLS;      // q (and k) elements a thread brings per stage
  const int s = blockIdx.x, h = blockIdx.y;
  const int tx = threadIdx.x, ty = threadIdx.y, NS = blockDim.y;
  const int tid = ty * MLSTM_COLS + tx, nthreads = MLSTM_COLS * NS;
  const int dpad = NS * ROWS;                 // = nthreads * ROWS / 32
  float* q_s = dyn_smem;                            // [TOK][dpad], zero beyond dim
  float* k_s = q_s + MLSTM_TOK * dpad;              // [TOK][dpad]
  float* v_s = k_s + MLSTM_TOK * dpad;              // [TOK][COLS] the tile's values times exp(i - m_t); the normaliser column: that factor
  float* red_s = v_s + MLSTM_TOK * MLSTM_COLS;      // [TOK][NS][COLS] partial read-outs
  float* keep_s = red_s + MLSTM_TOK * NS * MLSTM_COLS;      // [TOK] exp(f + m_(t-1) - m_t)
  const int row0 = seq_row0[s], len = seq_row0[s + 1] - row0, pos0 = seq_pos0[s];
  const int col = blockIdx.z * MLSTM_COLS + tx;     // 0 .. vdim (vdim: the normaliser)
  const bool live = col <= a.vdim;
  const int cols = a.vdim + 1;
  float* slot = a.state + (long long)seq_slot[s] * a.slot_stride + (long long)h * (a.dim + 1) * cols;
  float S[ROWS];
#pragma unroll
  for (int dd = 0; dd < ROWS; ++dd) {
    const int d = ty * ROWS + dd;
    S[dd] = (pos0 > 0 && live && d < a.dim) ? slot[(long long)d * cols + col] : 0.f;
  }
  // the next stage's operands travel from global memory into registers while the current stage computes.  Element tid + j * nthreads
  // of a stage's [TOK][dpad] block is token tid / dpad + (32 / ROWS) j, row tid % dpad: a thread keeps its row and walks the tokens.
  const int f_t = tid / dpad, f_d = tid % dpad;
  float pq[PF], pk[PF], pv[MLSTM_TOK / 2], pkeep = 0.f;      // at least two row groups: 8 tokens' values each at most
  auto fetch = [&](int c0) {
    const int nt = len - c0 < MLSTM_TOK ? len - c0 : MLSTM_TOK;
    const float* base = a.proj + (long long)(row0 + c0) * a.ld + h * a.dim + (f_d < a.dim ? f_d : 0);
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      const int t = f_t + (MLSTM_COLS / ROWS) * j;
      const bool ok = t < nt && f_d < a.dim;
      const float* row = base + (long long)(ok ? t : 0) * a.ld;
      pq[j] = ok ? row[a.q_off] * a.q_scale : 0.f;
      pk[j] = ok ? row[a.k_off] : 0.f;
    }
#pragma unroll
    for (int j = 0; j < MLSTM_TOK / 2; ++j) {      // thread (tx, ty) brings column tx of tokens ty, ty + NS, ...
      const int t = ty + j * NS;
      if (t < MLSTM_TOK) {
        float v = 0.f;
        if (t < nt && live) {
          const float take = gates[((long long)(row0 + c0 + t) * a.heads + h) * 3 + 1];
          v = col < a.vdim ? take * a.proj[(long long)(row0 + c0 + t) * a.ld + a.v_off + h * a.vdim + col] : take;
        }
        pv[j] = v;
      }
    }
    if (tid < MLSTM_TOK) pkeep = tid < nt ? gates[((long long)(row0 + c0 + tid) * a.heads + h) * 3] : 1.f;
  };
  fetch(0);
  for (int c0 = 0; c0 < len; c0 += MLSTM_TOK) {
    const int nt = len - c0 < MLSTM_TOK ? len - c0 : MLSTM_TOK;
    __syncthreads();      // the previous stage has been read
#pragma unroll
    for (int j = 0; j < PF; ++j) {
      q_s[tid + j * nthreads] = pq[j];
      k_s[tid + j * nthreads] = pk[j];
    }
#pragma unroll
    for (int j = 0; j < MLSTM_TOK / 2; ++j) {
      const int t = ty + j * NS;
      if (t < MLSTM_TOK) v_s[t * MLSTM_COLS + tx] = pv[j];
    }
    if (tid < MLSTM_TOK) keep_s[tid] = pkeep;
    __syncthreads();
    if (c0 + MLSTM_TOK < len) fetch(c0 + MLSTM_TOK);
#pragma unroll 4
    for (int t = 0; t < nt; ++t) {
      const float keep = keep_s[t], kv = v_s[t * MLSTM_COLS + tx];
      const float* kq = k_s + t * dpad + ty * ROWS;
      const float* qq = q_s + t * dpad + ty * ROWS;
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int dd = 0; dd < ROWS; dd += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(kq + dd);
        const float4 q4 = *reinterpret_cast<const float4*>(qq + dd);
        S[dd] = fmaf(keep, S[dd], k4.x * kv);
        S[dd + 1] = fmaf(keep, S[dd + 1], k4.y * kv);
        S[dd + 2] = fmaf(keep, S[dd + 2], k4.z * kv);
        S[dd + 3] = fmaf(keep, S[dd + 3], k4.w * kv);
        a0 = fmaf(S[dd], q4.x, a0);
        a1 = fmaf(S[dd + 1], q4.y, a1);
        a2 = fmaf(S[dd + 2], q4.z, a2);
        a3 = fmaf(S[dd + 3], q4.w, a3);
      }
      red_s[(t * NS + ty) * MLSTM_COLS + tx] = (a0 + a1) + (a2 + a3);
    }
    __syncthreads();
    // the row groups' partial read-outs, summed in their order: thread (tx, ty) takes column tx of tokens ty, ty + NS, ...
    if (live) {
      for (int t = ty; t < nt; t += NS) {
        float v = 0.f;
        for (int y = 0; y < NS; ++y) v += red_s[(t * NS + y) * MLSTM_COLS + tx];
        num[((long long)(row0 + c0 + t) * a.heads + h) * cols + col] = v;
      }
    }
  }
  if (live) {
#pragma unroll
    for (int dd = 0; dd < ROWS; ++dd) {
      const int d = ty * ROWS + dd;
      if (d < a.dim) slot[(long long)d * cols + col] = S[dd];
    }
  }
}

constexpr int MLSTM_FIN_WARPS = 4;
__global__ void __launch_bounds__(MLSTM_FIN_WARPS * 32)
mlstm_finish_kernel(MlstmArgs a, int R, const float* __restrict__ num, const float* __restrict__ gates) {
  const int item = blockIdx.x * MLSTM_FIN_WARPS + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (item >= R * a.heads) return;
  const int r = item / a.heads, h = item % a.heads;
  const int cols = a.vdim + 1;
  const float* nr = num + (long long)item * cols;
  const float den = fmaxf(fabsf(nr[a.vdim]), expf(-gates[(long long)item * 3 + 2])) + 1e-6f;
  float ss = 0.f;
  for (int c = lane; c < a.vdim; c += 32) {
    const float o = nr[c] / den;
    ss = fmaf(o, o, ss);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
  const float inv = 1.0f / sqrtf(ss / (float)a.vdim + a.eps);
  const float* g = a.proj + (long long)r * a.ld + a.g_off + h * a.vdim;
  for (int c = lane; c < a.vdim; c += 32) {
    float v = nr[c] / den * inv;
    if (a.out_gain != nullptr) v *= a.out_gain[h * a.vdim + c];
    v *= 1.0f / (1.0f + expf(-g[c]));
    const long long at = (long long)r * a.ldo + h * a.vdim + c;
    if (a.out_fp32) reinterpret_cast<float*>(a.out)[at] = v;
    else reinterpret_cast<bf16*>(a.out)[at] = __float2bfloat16(v);
  }
}

}  // namespace lp

using namespace lp;

extern "C" size_t lp_mlstm_workspace_bytes(int rows, int heads, int vdim) {
  return (size_t)rows * heads * (vdim + 1 + 3) * sizeof(float);
}

extern "C" int lp_mlstm(const lp_mlstm_desc* d, int n_seqs, int R, const int* seq_row0, const int* seq_pos0, const int* seq_slot,
                        void* ws, size_t ws_bytes, void* stream_) {
  cudaStream_t stream = reinterpret_cast<cudaStream_t>(stream_);
  LP_REQUIRE(d != nullptr && d->proj != nullptr && d->i_bias != nullptr && d->f_bias != nullptr && d->state != nullptr && d->out != nullptr,
             "lp_mlstm: null operand");
  LP_REQUIRE(d->heads > 0 && d->dim > 0 && d->vdim > 0 && d->dim <= MLSTM_MAX_GROUPS * MLSTM_ROWS,
             "lp_mlstm: bad sizes heads=%d dim=%d (at most %d) vdim=%d", d->heads, d->dim, MLSTM_MAX_GROUPS * MLSTM_ROWS, d->vdim);
  LP_REQUIRE(d->gate_cap > 0.f, "lp_mlstm: gate_cap must be positive");
  LP_REQUIRE(d->slot_stride >= (long long)d->heads * (d->dim + 1) * (d->vdim + 1), "lp_mlstm: a slot is smaller than the state");
  LP_REQUIRE(seq_row0 != nullptr && seq_pos0 != nullptr && seq_slot != nullptr && n_seqs >= 0 && R >= 0, "lp_mlstm: bad batch tables");
  if (n_seqs == 0 || R == 0) return 0;
  LP_REQUIRE(ws != nullptr && ws_bytes >= lp_mlstm_workspace_bytes(R, d->heads, d->vdim), "lp_mlstm: workspace too small");
  MlstmArgs a;
  a.proj = d->proj; a.ld = d->ld; a.q_off = d->q_off; a.k_off = d->k_off; a.v_off = d->v_off; a.g_off = d->g_off; a.i_off = d->i_off;
  a.f_off = d->f_off; a.heads = d->heads; a.dim = d->dim; a.vdim = d->vdim; a.i_bias = d->i_bias; a.f_bias = d->f_bias;
  a.gate_cap = d->gate_cap; a.q_scale = d->q_scale; a.eps = d->eps; a.out_gain = d->out_gain; a.state = d->state;
  a.slot_stride = d->slot_stride; a.out = d->out; a.ldo = d->ldo; a.out_fp32 = d->out_fp32;
  float* num = reinterpret_cast<float*>(ws);
  float* gates = num + (size_t)R * d->heads * (d->vdim + 1);
  const int rows = d->dim <= 8 * MLSTM_MAX_GROUPS ? 8 : MLSTM_ROWS;
  const int ns = d->dim <= rows ? 2 : (d->dim + rows - 1) / rows;      // at least two row groups (rows past dim stay zero)
  const size_t smem = ((size_t)2 * MLSTM_TOK * ns * rows + MLSTM_TOK * MLSTM_COLS + (size_t)MLSTM_TOK * ns * MLSTM_COLS + MLSTM_TOK) *
                      sizeof(float);
  static size_t have8 = 48 * 1024, have16 = 48 * 1024;      // raised once per instantiation, and only for head sizes that need it
  size_t& have = rows == 8 ? have8 : have16;
  if (smem > have) {
    if (rows == 8) LP_CHECK_CUDA(cudaFuncSetAttribute(mlstm_scan_kernel<8>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    else LP_CHECK_CUDA(cudaFuncSetAttribute(mlstm_scan_kernel<MLSTM_ROWS>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024));
    have = 96 * 1024;
  }
  mlstm_gate_kernel<<<n_seqs * d->heads, MLSTM_GATE_WARPS * 32, 0, stream>>>(
      a, n_seqs, seq_row0, seq_pos0, seq_slot, gates);
  LP_CHECK_CUDA(cudaGetLastError());
  const dim3 grid(n_seqs, d->heads, (d->vdim + 1 + MLSTM_COLS - 1) / MLSTM_COLS);
  if (rows == 8) mlstm_scan_kernel<8><<<grid, dim3(MLSTM_COLS, ns), smem, stream>>>(a, seq_row0, seq_pos0, seq_slot, gates, num);
  else mlstm_scan_kernel<MLSTM_ROWS><<<grid, dim3(MLSTM_COLS, ns), smem, stream>>>(a, seq_row0, seq_pos0, seq_slot, gates, num);
  LP_CHECK_CUDA(cudaGetLastError());
  mlstm_finish_kernel<<<(R * d->heads + MLSTM_FIN_WARPS - 1) / MLSTM_FIN_WARPS, MLSTM_FIN_WARPS * 32, 0, stream>>>(a, R, num, gates);
  LP_CHECK_CUDA(cudaGetLastError());
  note_launch(3);
  return 0;
}
