// Kernels for layers whose branches run side by side (x += mixer(N1 x) + ff(N2 x)), for attention with
// per-head norms and a partial rotation, for a recurrent mixer with a matrix state, and for routed experts.
//
//   tanh_norm          resid += sum of pending branch outputs (each a [N, W] array or a K-split stack, each with
//                      a scale) (+ one broadcast row); then up to two norms of the same row,
//                      out_k = tanh(alpha_k x) * w_k + b_k; or the same on a few gathered rows
//   head_prep          a fused q|k|v|gate projection: bias, RMS norm per head with one weight for all heads,
//                      rotation of each head's first dimensions, q to its buffer, k and v into their pages
//                      (heads padded to the kernels' head size), sigmoid of the per-head gate
//   matrix_memory_scan the recurrence S_t = keep_t S_(t-1) + take_t k_t v_t^T of a matrix-memory mixer, token by
//                      token with the state on chip, for portions and single tokens alike
//   matrix_memory_out  its outputs: divided by their denominator, each head over its root mean square, times a
//                      weight and a sigmoid gate
//   route_top          router logits, softmax over all experts, the `top` largest renormalised, as a dense
//                      [N, experts (+ 1)] array of weights (0 where an expert is not chosen), the shared expert's
//                      sigmoid gate in the last column
//   act_mul_blocks     act(gate) * up * the weight of the column's expert
//
// Norms, gates, decays, states, routers and the residual sum are float32; a result is rounded once, when it is
// stored in the activation type.
#include "common.cuh"

namespace parallel {

constexpr int MAX_TERMS = 4;

struct SumTerm {
  const float* data;      // [partials][N][W]
  long long stride;       // elements between partials
  int partials;
  float scale;
};

struct TanhNormArgs {
  float* resid;           // [N][W]
  SumTerm terms[MAX_TERMS];
  int num_terms;
  const float* row_add;   // [W] or null: added to every row
  const int* rows;        // null: every row, the residual is rewritten; else out[r] = norm(x[rows[r]]), nothing else written
  int norms;              // 0, 1 or 2
  float alpha[2];
  const float* weight[2];
  const float* bias[2];
  void* out[2];
  int n, width;
};

// tanh in the activation type's accuracy: bfloat16 results keep 8 bits, so the hardware exponential serves
// (absolute error about 1e-7); float32 uses tanhf.
template <typename T> __device__ __forceinline__ float tanh_for(float z);
template <> __device__ __forceinline__ float tanh_for<float>(float z) { return tanhf(z); }
template <> __device__ __forceinline__ float tanh_for<__nv_bfloat16>(float z) {
  const float c = fminf(fmaxf(z, -15.f), 15.f);
  return 1.0f - __fdividef(2.0f, __expf(2.0f * c) + 1.0f);
}

template <typename TO, int VEC>
__global__ void __launch_bounds__(256) tanh_norm_kernel(const TanhNormArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int groups = a.width / VEC;
  for (int row = blockIdx.y; row < a.n; row += gridDim.y) {
    const int src = a.rows != nullptr ? a.rows[row] : row;
    const size_t src_base = static_cast<size_t>(src) * a.width, out_base = static_cast<size_t>(row) * a.width;
    for (int group = blockIdx.x * blockDim.x + threadIdx.x; group < groups; group += gridDim.x * blockDim.x) {
      const int col = group * VEC;
      float x[VEC];
#pragma unroll
      for (int e = 0; e < VEC; ++e) x[e] = a.resid[src_base + col + e];
      for (int t = 0; t < a.num_terms; ++t) {
        const SumTerm& term = a.terms[t];
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          x[e] = __fmaf_rn(term.scale, sum_partials(term.data + src_base + col + e, term.stride, term.partials), x[e]);
      }
      if (a.row_add != nullptr) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) x[e] = __fadd_rn(x[e], a.row_add[col + e]);
      }
      if (a.rows == nullptr && (a.num_terms > 0 || a.row_add != nullptr)) {
#pragma unroll
        for (int e = 0; e < VEC; ++e) a.resid[src_base + col + e] = x[e];
      }
      for (int k = 0; k < a.norms; ++k) {
        TO* out = static_cast<TO*>(a.out[k]) + out_base + col;
#pragma unroll
        for (int e = 0; e < VEC; ++e)
          out[e] = from_float<TO>(__fmaf_rn(tanh_for<TO>(a.alpha[k] * x[e]), a.weight[k][col + e], a.bias[k][col + e]));
      }
    }
  }
}

// ---------------------------------------------------------------------------------------------- head_prep
struct HeadPrepArgs {
  const float* fused;     // [partials][N][total]: q (H D) | k (G D) | v (G Dv) | gate (H, when gate_out)
  long long stride;
  int partials, total;
  const float* bias;      // [total] or null
  const int* positions;   // [N]
  const float* inv_freq;  // [rot / 2] or null
  int rot;                // rotated dimensions of a head (even, <= D); 0: none
  const float* q_weight;  // [D] or null
  const float* k_weight;  // [D] or null
  float eps;
  void* q_out;            // [N][H][Dp]
  void* keys;             // [slots][G][Dp] or null
  void* values;           // [slots][G][Dp]
  const int* slots;       // [N]; -1: nothing is stored
  float* gate_out;        // [N][H] or null
  int n, heads, kv_heads, dim, vdim, padded, num_slots;
};

constexpr int PREP_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32) head_prep_kernel(const HeadPrepArgs a) {
  extern __shared__ float prep_shared[];
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int units = a.heads + 2 * a.kv_heads + (a.gate_out != nullptr ? 1 : 0);
  const long long work = static_cast<long long>(blockIdx.x) * PREP_WARPS + warp;
  if (work >= static_cast<long long>(a.n) * units) return;
  const int token = static_cast<int>(work / units), unit = static_cast<int>(work - static_cast<long long>(token) * units);
  const float* row = a.fused + static_cast<size_t>(token) * a.total;
  const int q_cols = a.heads * a.dim, k_cols = a.kv_heads * a.dim, v_cols = a.kv_heads * a.vdim;
  if (unit == a.heads + 2 * a.kv_heads) {   // the gates: one number a head
    for (int h = lane; h < a.heads; h += 32) {
      const int col = q_cols + k_cols + v_cols + h;
      float z = sum_partials(row + col, a.stride, a.partials);
      if (a.bias != nullptr) z = __fadd_rn(z, a.bias[col]);
      a.gate_out[static_cast<size_t>(token) * a.heads + h] = 1.0f / (1.0f + expf(-z));
    }
    return;
  }
  const bool is_q = unit < a.heads, is_k = !is_q && unit < a.heads + a.kv_heads;
  const int head = is_q ? unit : (is_k ? unit - a.heads : unit - a.heads - a.kv_heads);
  const int size = (is_q || is_k) ? a.dim : a.vdim;
  const int first_col = is_q ? head * a.dim : (is_k ? q_cols + head * a.dim : q_cols + k_cols + head * a.vdim);
  const int slot = a.slots[token];
  T* dst;
  if (is_q) dst = static_cast<T*>(a.q_out) + (static_cast<size_t>(token) * a.heads + head) * a.padded;
  else {
    if (a.keys == nullptr || slot < 0 || slot >= a.num_slots) return;
    dst = static_cast<T*>(is_k ? a.keys : a.values) + (static_cast<size_t>(slot) * a.kv_heads + head) * a.padded;
  }
  float* mine = prep_shared + static_cast<size_t>(warp) * a.padded;
  float squares = 0.f;
  for (int d = lane; d < size; d += 32) {
    float v = sum_partials(row + first_col + d, a.stride, a.partials);
    if (a.bias != nullptr) v = __fadd_rn(v, a.bias[first_col + d]);
    mine[d] = v;
    squares = __fmaf_rn(v, v, squares);
  }
  const float* weight = is_q ? a.q_weight : (is_k ? a.k_weight : nullptr);
  if (weight != nullptr) {
    const float r = rsqrtf(warp_sum(squares) / static_cast<float>(size) + a.eps);
    for (int d = lane; d < size; d += 32) mine[d] = mine[d] * r * weight[d];
  }
  __syncwarp();
  const int half = (is_q || is_k) && a.inv_freq != nullptr ? a.rot / 2 : 0;
  const float position = static_cast<float>(a.positions[token]);
  for (int d = lane; d < a.padded; d += 32) {
    float v = d < size ? mine[d] : 0.f;
    if (d < 2 * half) {
      const int i = d < half ? d : d - half;
      float sine, cosine;
      sincosf(__fmul_rn(position, a.inv_freq[i]), &sine, &cosine);
      const float u = mine[i], w = mine[i + half];
      v = d < half ? __fsub_rn(__fmul_rn(u, cosine), __fmul_rn(w, sine)) : __fadd_rn(__fmul_rn(w, cosine), __fmul_rn(u, sine));
    }
    dst[d] = from_float<T>(v);
  }
}

// ------------------------------------------------------------------------------------- matrix memory: scan
// One CTA owns `cols` value columns of one head's state for one sequence and walks the sequence's new tokens in
// order.  Thread j holds column j: S[:, j] lives in shared memory as S[d * ld + j].  The normaliser z (the
// recurrence with v = 1) is one more column, kept by the CTA of the head's first columns.  Tokens are staged
// TOKENS at a time (q, k, this CTA's v columns, the two gates), so the walk itself touches shared memory only.
// The state of a slot: per head D * Dv floats of S (row d, column j at d * Dv + j), D of z, then m.
struct ScanArgs {
  const float* fused;     // [partials][N][total]: q (H D) | k (H D) | v (H Dv) | gate (H Dv) | i (H) | f (H)
  long long stride;
  int partials, total;
  const float* gate_bias; // [2 H]: input gates, then forget gates; or null
  float* state;           // [slots][H][D Dv + D + 1]
  const int* q_start;     // [S + 1]
  const int* state_slot;  // [S]; -1: the sequence is padding
  float* numerator;       // [N][H][Dv]
  float* denominator;     // [N][H]
  int heads, dim, vdim, cols, num_slots;
  float cap, q_scale, floor_;
};

constexpr int SCAN_TOKENS = 8;

__device__ __forceinline__ float log_sigmoid(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

__global__ void matrix_memory_scan_kernel(const ScanArgs a) {
  extern __shared__ float scan_shared[];
  let_dependents_start();
  wait_for_previous();
  const int seq = blockIdx.z, head = blockIdx.y, col0 = blockIdx.x * a.cols;
  const int slot = a.state_slot[seq];
  const int start = a.q_start[seq], count = a.q_start[seq + 1] - start;
  const int cols_here = min(a.cols, a.vdim - col0);
  if (slot < 0 || slot >= a.num_slots) {
    // a padding row of the batch: no state is touched; its outputs are made finite (0 over 1) for the kernels after
    for (int idx = threadIdx.x; idx < count * cols_here; idx += blockDim.x) {
      const int t = idx / cols_here, c = idx - t * cols_here;
      a.numerator[(static_cast<size_t>(start + t) * a.heads + head) * a.vdim + col0 + c] = 0.f;
    }
    if (blockIdx.x == 0)
      for (int t = threadIdx.x; t < count; t += blockDim.x) a.denominator[static_cast<size_t>(start + t) * a.heads + head] = 1.f;
    return;
  }
  const bool keeps_z = blockIdx.x == 0;
  const int ld = a.cols + 1;
  const int D = a.dim, Dv = a.vdim, H = a.heads;
  float* S = scan_shared;                           // [D][ld]
  float* qs = S + static_cast<size_t>(D) * ld;      // [TOKENS][D]
  float* ks = qs + SCAN_TOKENS * D;                 // [TOKENS][D]
  float* vs = ks + SCAN_TOKENS * D;                 // [TOKENS][cols]
  float* gates = vs + SCAN_TOKENS * a.cols;         // [TOKENS][2]: input gate, log forget gate
  float* mine = a.state + (static_cast<size_t>(slot) * H + head) * (static_cast<size_t>(D) * Dv + D + 1);
  for (int idx = threadIdx.x; idx < D * cols_here; idx += blockDim.x) {
    const int d = idx / cols_here, j = idx - d * cols_here;
    S[d * ld + j] = mine[static_cast<size_t>(d) * Dv + col0 + j];
  }
  if (keeps_z)
    for (int d = threadIdx.x; d < D; d += blockDim.x) S[d * ld + a.cols] = mine[static_cast<size_t>(D) * Dv + d];
  float m = mine[static_cast<size_t>(D) * Dv + D];
  const int j = threadIdx.x;
  const bool value_column = j < cols_here, z_column = keeps_z && j == a.cols;
  const int q_cols = H * D, v_first = 2 * q_cols, gate_first = 2 * q_cols + 2 * H * Dv;
  for (int t0 = 0; t0 < count; t0 += SCAN_TOKENS) {
    const int here = min(SCAN_TOKENS, count - t0);
    __syncthreads();
    for (int idx = threadIdx.x; idx < here * D; idx += blockDim.x) {
      const int t = idx / D, d = idx - t * D;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      qs[t * D + d] = __fmul_rn(sum_partials(row + head * D + d, a.stride, a.partials), a.q_scale);
      ks[t * D + d] = sum_partials(row + q_cols + head * D + d, a.stride, a.partials);
    }
    for (int idx = threadIdx.x; idx < here * cols_here; idx += blockDim.x) {
      const int t = idx / cols_here, c = idx - t * cols_here;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      vs[t * a.cols + c] = sum_partials(row + v_first + head * Dv + col0 + c, a.stride, a.partials);
    }
    for (int idx = threadIdx.x; idx < here * 2; idx += blockDim.x) {
      const int t = idx >> 1, which = idx & 1;
      const float* row = a.fused + static_cast<size_t>(start + t0 + t) * a.total;
      float z = sum_partials(row + gate_first + which * H + head, a.stride, a.partials);
      if (a.gate_bias != nullptr) z = __fadd_rn(z, a.gate_bias[which * H + head]);
      z = a.cap * tanhf(z / a.cap);
      gates[t * 2 + which] = which == 0 ? z : log_sigmoid(z);
    }
    __syncthreads();
    for (int t = 0; t < here; ++t) {
      const float gate_in = gates[t * 2], gate_forget = gates[t * 2 + 1];
      const float m_new = fmaxf(gate_forget + m, gate_in);
      const float keep = expf(gate_forget + m - m_new), take = expf(gate_in - m_new);
      m = m_new;
      if (value_column || z_column) {
        const float tv = z_column ? take : __fmul_rn(take, vs[t * a.cols + j]);
        const float* q = qs + t * D;
        const float* k = ks + t * D;
        float acc = 0.f;
        for (int d = 0; d < D; ++d) {
          const float s = __fmaf_rn(tv, k[d], __fmul_rn(keep, S[d * ld + j]));
          S[d * ld + j] = s;
          acc = __fmaf_rn(s, q[d], acc);
        }
        const size_t token = static_cast<size_t>(start + t0 + t);
        if (z_column) a.denominator[token * H + head] = fmaxf(fabsf(acc), expf(-m)) + a.floor_;
        else a.numerator[(token * H + head) * Dv + col0 + j] = acc;
      }
    }
  }
  __syncthreads();
  for (int idx = threadIdx.x; idx < D * cols_here; idx += blockDim.x) {
    const int d = idx / cols_here, c = idx - d * cols_here;
    mine[static_cast<size_t>(d) * Dv + col0 + c] = S[d * ld + c];
  }
  if (keeps_z) {
    for (int d = threadIdx.x; d < D; d += blockDim.x) mine[static_cast<size_t>(D) * Dv + d] = S[d * ld + a.cols];
    if (threadIdx.x == 0) mine[static_cast<size_t>(D) * Dv + D] = m;
  }
}

// -------------------------------------------------------------------------------------- matrix memory: out
struct MemoryOutArgs {
  const float* numerator;    // [N][H][Dv]
  const float* denominator;  // [N][H]
  const float* fused;        // the projection the scan read; its gate columns start at `gate_first`
  long long stride;
  int partials, total, gate_first;
  const float* weight;       // [H Dv]
  float eps;
  void* out;                 // [N][H Dv]
  int n, heads, vdim;
};

template <typename T>
__global__ void __launch_bounds__(PREP_WARPS * 32) matrix_memory_out_kernel(const MemoryOutArgs a) {
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const long long work = static_cast<long long>(blockIdx.x) * PREP_WARPS + warp;
  if (work >= static_cast<long long>(a.n) * a.heads) return;
  const int token = static_cast<int>(work / a.heads), head = static_cast<int>(work - static_cast<long long>(token) * a.heads);
  const float* num = a.numerator + static_cast<size_t>(work) * a.vdim;
  const float inv = 1.0f / a.denominator[work];
  float squares = 0.f;
  for (int c = lane; c < a.vdim; c += 32) {
    const float o = __fmul_rn(num[c], inv);
    squares = __fmaf_rn(o, o, squares);
  }
  const float r = rsqrtf(warp_sum(squares) / static_cast<float>(a.vdim) + a.eps);
  const float* gate_row = a.fused + static_cast<size_t>(token) * a.total + a.gate_first + head * a.vdim;
  T* out = static_cast<T*>(a.out) + (static_cast<size_t>(token) * a.heads + head) * a.vdim;
  for (int c = lane; c < a.vdim; c += 32) {
    const float gate = 1.0f / (1.0f + expf(-sum_partials(gate_row + c, a.stride, a.partials)));
    out[c] = from_float<T>(__fmul_rn(num[c], inv) * r * a.weight[head * a.vdim + c] * gate);
  }
}

// ----------------------------------------------------------------------------------------------- route_top
constexpr int ROUTE_WARPS = 4;

template <typename T>
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
route_top_kernel(const T* __restrict__ x, const float* __restrict__ router, const float* __restrict__ shared_gate,
                 float* __restrict__ weights, int n, int width, int experts, int top, int columns, float renorm_eps) {
  extern __shared__ float route_shared[];
  let_dependents_start();
  wait_for_previous();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int token = blockIdx.x * ROUTE_WARPS + warp;
  if (token >= n) return;
  float* score = route_shared + static_cast<size_t>(warp) * experts;
  const T* row = x + static_cast<size_t>(token) * width;
  float* out = weights + static_cast<size_t>(token) * columns;
  float best = -INFINITY;
  for (int e = 0; e < experts; ++e) {
    const float* w = router + static_cast<size_t>(e) * width;
    float dot = 0.f;
    for (int c = lane; c < width; c += 32) dot = __fmaf_rn(to_float(row[c]), w[c], dot);
    dot = warp_sum(dot);
    if (lane == 0) score[e] = dot;
    best = fmaxf(best, dot);
  }
  __syncwarp();
  float total = 0.f;
  for (int e = lane; e < experts; e += 32) {
    const float p = expf(score[e] - best);
    score[e] = p;
    total += p;
  }
  total = warp_sum(total);
  __syncwarp();
  for (int e = lane; e < experts; e += 32) {
    score[e] = score[e] / total;
    out[e] = 0.f;
  }
  __syncwarp();
  float chosen_sum = 0.f;
  // `top` rounds of a warp-wide argmax; the lowest index wins a tie.  A pick is marked by negating its score.
  for (int round = 0; round < top; ++round) {
    float mine = -1.f;
    int where = experts;
    for (int e = lane; e < experts; e += 32)
      if (score[e] > mine) { mine = score[e]; where = e; }
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, mine, offset);
      const int other_where = __shfl_xor_sync(0xffffffffu, where, offset);
      if (other > mine || (other == mine && other_where < where)) { mine = other; where = other_where; }
    }
    chosen_sum += mine;
    if (lane == 0 && where < experts) {
      out[where] = mine;
      score[where] = -2.f;
    }
    __syncwarp();
  }
  const float inv = 1.0f / (chosen_sum + renorm_eps);
  for (int e = lane; e < experts; e += 32) out[e] = out[e] * inv;
  if (columns > experts) {
    float gate = 1.f;
    if (shared_gate != nullptr) {
      float dot = 0.f;
      for (int c = lane; c < width; c += 32) dot = __fmaf_rn(to_float(row[c]), shared_gate[c], dot);
      gate = 1.0f / (1.0f + expf(-warp_sum(dot)));
    }
    if (lane == 0) out[experts] = gate;
  }
}

// ------------------------------------------------------------------------------------------ act_mul_blocks
// gate_up [N][2 I]: all gate columns, then all up columns; I = experts * each + rest.  Column c belongs to
// expert c / each, the last `rest` columns to the shared expert (weight column `experts`).
template <typename T>
__global__ void __launch_bounds__(256)
act_mul_blocks_kernel(const T* __restrict__ gate_up, const float* __restrict__ weights, T* __restrict__ out, int n, int inter,
                      int experts, int each, int columns, int act, float limit) {
  let_dependents_start();
  wait_for_previous();
  for (int row = blockIdx.y; row < n; row += gridDim.y) {
    const T* in = gate_up + static_cast<size_t>(row) * 2 * inter;
    const float* w = weights + static_cast<size_t>(row) * columns;
    T* o = out + static_cast<size_t>(row) * inter;
    for (int c = blockIdx.x * blockDim.x + threadIdx.x; c < inter; c += gridDim.x * blockDim.x) {
      const int block = c < experts * each ? c / each : experts;
      const float share = w[block];
      // an expert the token did not choose contributes exactly nothing, whatever its gate and up columns hold
      const float y = share == 0.f ? 0.f : __fmul_rn(act_times<T>(act, to_float(in[c]), to_float(in[inter + c]), limit), share);
      o[c] = from_float<T>(y);
    }
  }
}

}  // namespace parallel

// =========================================================================================== launchers
using namespace parallel;

// terms: `num_terms` (at most 4) pending sums, term t = data[t] ([partials[t]][N][W] float32, `strides[t]` elements
// between partials) times scales[t].  norms: 0..2, norm k = tanh(alpha[k] x) * weight[k] + bias[k] into out[k]
// ([N or R][W] of out_dtype).  rows null: resid is rewritten with the sum; else only out[k][r] for row rows[r].
SHRIKE_API int shrike_tanh_norm(float* resid, const float* const* data, const int* partials, const long long* strides,
                                const float* scales, int num_terms, const float* row_add, const int* rows, int norms,
                                const float* alpha, const float* const* weight, const float* const* bias, void* const* out,
                                int out_dtype, int n, int width, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (width <= 0 || num_terms < 0 || num_terms > MAX_TERMS || norms < 0 || norms > 2) return SHRIKE_BAD_ARGUMENT;
  if (norms > 0 && out_dtype != SHRIKE_F32 && out_dtype != SHRIKE_BF16) return SHRIKE_BAD_ARGUMENT;
  TanhNormArgs a = {};
  a.resid = resid;
  a.num_terms = num_terms;
  for (int t = 0; t < num_terms; ++t) {
    if (partials[t] < 1) return SHRIKE_BAD_ARGUMENT;
    a.terms[t] = SumTerm{data[t], strides[t], partials[t], scales[t]};
  }
  a.row_add = row_add;
  a.rows = rows;
  a.norms = norms;
  for (int k = 0; k < norms; ++k) {
    a.alpha[k] = alpha[k];
    a.weight[k] = weight[k];
    a.bias[k] = bias[k];
    a.out[k] = out[k];
  }
  a.n = n;
  a.width = width;
  const bool vec = width % 4 == 0;
  const int groups = vec ? width / 4 : width;
  const dim3 grid(max(1, min(32, (groups + 255) / 256)), max(1, min(n, 65535)));
  const bool bf16 = norms > 0 && out_dtype == SHRIKE_BF16;
  if (vec && bf16) launch_dependent(tanh_norm_kernel<__nv_bfloat16, 4>, grid, 256, 0, stream, a);
  else if (vec) launch_dependent(tanh_norm_kernel<float, 4>, grid, 256, 0, stream, a);
  else if (bf16) launch_dependent(tanh_norm_kernel<__nv_bfloat16, 1>, grid, 256, 0, stream, a);
  else launch_dependent(tanh_norm_kernel<float, 1>, grid, 256, 0, stream, a);
  return shrike_launch_status();
}

SHRIKE_API int shrike_head_prep(const float* fused, int partials, long long stride, int total, const float* bias,
                                const int* positions, const float* inv_freq, int rot, const float* q_weight,
                                const float* k_weight, float eps, void* q_out, void* keys, void* values, const int* slots,
                                float* gate_out, int dtype, int n, int heads, int kv_heads, int dim, int vdim, int padded,
                                int num_slots, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads < 1 || kv_heads < 1 || dim < 1 || vdim < 1 || padded < dim || padded < vdim || partials < 1 || rot < 0 ||
      rot % 2 || rot > dim || padded > 8192)
    return SHRIKE_BAD_ARGUMENT;
  if (total < heads * dim + kv_heads * (dim + vdim) + (gate_out != nullptr ? heads : 0)) return SHRIKE_BAD_ARGUMENT;
  HeadPrepArgs a = {fused, stride, partials, total, bias, positions, inv_freq, rot, q_weight, k_weight, eps, q_out, keys,
                    values, slots, gate_out, n, heads, kv_heads, dim, vdim, padded, num_slots};
  const int units = heads + 2 * kv_heads + (gate_out != nullptr ? 1 : 0);
  const long long work = static_cast<long long>(n) * units;
  const unsigned blocks = static_cast<unsigned>((work + PREP_WARPS - 1) / PREP_WARPS);
  const size_t smem = static_cast<size_t>(PREP_WARPS) * padded * sizeof(float);
  if (dtype == SHRIKE_F32) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_prep_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_dependent(head_prep_kernel<float>, blocks, PREP_WARPS * 32, smem, stream, a);
  } else if (dtype == SHRIKE_BF16) {
    if (smem > 48 * 1024) cudaFuncSetAttribute(head_prep_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
    launch_dependent(head_prep_kernel<__nv_bfloat16>, blocks, PREP_WARPS * 32, smem, stream, a);
  } else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

// Value columns a CTA of the scan takes: as many (at most 64) as let the state slice, the staged tokens and a
// second CTA fit an SM's shared memory.
static int scan_columns(int dim, int vdim, size_t* smem_out) {
  const ShrikeDevice& device = shrike_device();
  int cols = vdim < 64 ? vdim : 64;
  for (;;) {
    const size_t floats = static_cast<size_t>(dim) * (cols + 1) + 2ull * SCAN_TOKENS * dim + static_cast<size_t>(SCAN_TOKENS) * cols +
                          2 * SCAN_TOKENS;
    const size_t bytes = floats * sizeof(float);
    if (bytes <= static_cast<size_t>(device.max_smem) / 2 || cols <= 8) {
      *smem_out = bytes;
      return bytes <= static_cast<size_t>(device.max_smem) ? cols : 0;
    }
    cols = (cols + 1) / 2;
  }
}

SHRIKE_API int shrike_matrix_memory_scan(const float* fused, int partials, long long stride, int total, const float* gate_bias,
                                         float* state, const int* q_start, const int* state_slot, float* numerator,
                                         float* denominator, int num_seqs, int heads, int dim, int vdim, int num_slots,
                                         float cap, float q_scale, float floor_, cudaStream_t stream) {
  if (num_seqs <= 0) return SHRIKE_OK;
  if (heads < 1 || dim < 1 || vdim < 1 || partials < 1 || !(cap > 0.f) || num_seqs > 65535 || heads > 65535) return SHRIKE_BAD_ARGUMENT;
  if (total < 2 * heads * dim + 2 * heads * vdim + 2 * heads) return SHRIKE_BAD_ARGUMENT;
  size_t smem = 0;
  const int cols = scan_columns(dim, vdim, &smem);
  if (cols == 0) return SHRIKE_BAD_ARGUMENT;
  static size_t configured = 0;
  if (smem > 48 * 1024 && smem > configured) {
    const cudaError_t err = cudaFuncSetAttribute(matrix_memory_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                 shrike_device().max_smem);
    if (err != cudaSuccess) return static_cast<int>(err);
    configured = shrike_device().max_smem;
  }
  ScanArgs a = {fused, stride, partials, total, gate_bias, state, q_start, state_slot, numerator, denominator,
                heads, dim, vdim, cols, num_slots, cap, q_scale, floor_};
  const dim3 grid((vdim + cols - 1) / cols, heads, num_seqs);
  const int threads = (cols + 1 + 31) / 32 * 32;
  launch_dependent(matrix_memory_scan_kernel, grid, threads, smem, stream, a);
  return shrike_launch_status();
}

SHRIKE_API int shrike_matrix_memory_out(const float* numerator, const float* denominator, const float* fused, int partials,
                                        long long stride, int total, int gate_first, const float* weight, float eps, void* out,
                                        int dtype, int n, int heads, int vdim, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (heads < 1 || vdim < 1 || partials < 1 || gate_first < 0 || gate_first + heads * vdim > total) return SHRIKE_BAD_ARGUMENT;
  MemoryOutArgs a = {numerator, denominator, fused, stride, partials, total, gate_first, weight, eps, out, n, heads, vdim};
  const long long work = static_cast<long long>(n) * heads;
  const unsigned blocks = static_cast<unsigned>((work + PREP_WARPS - 1) / PREP_WARPS);
  if (dtype == SHRIKE_F32) launch_dependent(matrix_memory_out_kernel<float>, blocks, PREP_WARPS * 32, 0, stream, a);
  else if (dtype == SHRIKE_BF16) launch_dependent(matrix_memory_out_kernel<__nv_bfloat16>, blocks, PREP_WARPS * 32, 0, stream, a);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

// weights [N][columns], columns = experts (+ 1 when there is a shared expert: its gate, sigmoid(shared_gate . x), or 1
// when shared_gate is null).
SHRIKE_API int shrike_route_top(const void* x, int dtype, const float* router, const float* shared_gate, float* weights, int n,
                                int width, int experts, int top, int columns, float renorm_eps, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (experts < 1 || top < 1 || top > experts || experts > 2048 || (columns != experts && columns != experts + 1)) return SHRIKE_BAD_ARGUMENT;
  const unsigned blocks = static_cast<unsigned>((n + ROUTE_WARPS - 1) / ROUTE_WARPS);
  const size_t smem = static_cast<size_t>(ROUTE_WARPS) * experts * sizeof(float);
  if (dtype == SHRIKE_F32)
    launch_dependent(route_top_kernel<float>, blocks, ROUTE_WARPS * 32, smem, stream, static_cast<const float*>(x), router,
                     shared_gate, weights, n, width, experts, top, columns, renorm_eps);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(route_top_kernel<__nv_bfloat16>, blocks, ROUTE_WARPS * 32, smem, stream, static_cast<const __nv_bfloat16*>(x),
                     router, shared_gate, weights, n, width, experts, top, columns, renorm_eps);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}

SHRIKE_API int shrike_act_mul_blocks(const void* gate_up, const float* weights, void* out, int dtype, int n, int inter, int experts,
                                     int each, int columns, int act, float limit, cudaStream_t stream) {
  if (n <= 0) return SHRIKE_OK;
  if (inter < 1 || experts < 1 || each < 1 || experts * each > inter || !known_activation(act)) return SHRIKE_BAD_ARGUMENT;
  if (experts * each < inter && columns != experts + 1) return SHRIKE_BAD_ARGUMENT;
  const dim3 grid(max(1, min(64, (inter + 255) / 256)), max(1, min(n, 65535)));
  if (dtype == SHRIKE_F32)
    launch_dependent(act_mul_blocks_kernel<float>, grid, 256, 0, stream, static_cast<const float*>(gate_up), weights,
                     static_cast<float*>(out), n, inter, experts, each, columns, act, limit);
  else if (dtype == SHRIKE_BF16)
    launch_dependent(act_mul_blocks_kernel<__nv_bfloat16>, grid, 256, 0, stream, static_cast<const __nv_bfloat16*>(gate_up), weights,
                     static_cast<__nv_bfloat16*>(out), n, inter, experts, each, columns, act, limit);
  else return SHRIKE_BAD_ARGUMENT;
  return shrike_launch_status();
}
