// Recurrent mixers whose gates are ONE number per head and token, with a float32 state per request.
//
// Matrix memory (mLSTM).  Per head a matrix S [dim][vdim], a vector n [dim] and a running maximum m (all
// zero at the start of a request).  With a log input gate i_t and a log forget gate f_t,
//
//     i_t = cap * tanh((x_i + b_i) / cap)        f_t = logsigmoid(cap * tanh((x_f + b_f) / cap))
//     m_t = max(f_t + m_(t-1), i_t)
//     S_t = exp(f_t + m_(t-1) - m_t) S_(t-1) + exp(i_t - m_t) k_t v_t^T        (n_t the same with k_t alone)
//     o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + 1e-6)
//
// Gated delta rule.  Per head a matrix S [dim][vdim]; unit vectors k_t and q_t (x / sqrt(sum(x^2) + 1e-6), q
// also times a constant), a write strength b_t = sigmoid(x_b) and a decay
// g_t = exp(-exp(A) * softplus(x_a + dt)):
//
//     S <- g_t S;   u = b_t (v_t - S^T k_t);   S <- S + k_t u^T;   o_t = S^T q_t
//
// Its q, k and v first pass a short causal convolution over time per channel (the last tap multiplies the
// current token; the inputs of the last taps - 1 tokens are part of the request's state) and SiLU.
//
// Both scans: a block per (request, head, block of value columns); eight lanes share a value column, each
// keeps an eighth of its rows in registers, and their sums meet by shuffles.  The rows a token brings are
// staged in shared memory one token ahead.  Everything is float32.  A request's result depends on its own
// tokens and state only, whatever the batch, the cut of a prompt into portions, or the slot.
//
// A last kernel divides every head of a scan's output by its own root mean square, multiplies by a gain
// (one number per column, or a vector of a head's size shared by the heads) and by sigmoid or SiLU of a
// gate, and rounds once.
#include "common.cuh"

CIE_DEFINE_LAST_ERROR()

namespace cie {

constexpr int kLanes = 8;        // lanes that share a value column
constexpr int kScanMaxDim = 256;  // largest number of rows (key size) of a state matrix
constexpr int kMaxTaps = 16;     // longest short convolution
constexpr int kNormaliserColumns = 32;   // value columns that share one copy of the matrix memory's n and m

__device__ __forceinline__ float sigmoid_f(float z) { return 1.f / (1.f + expf(-z)); }
__device__ __forceinline__ float log_sigmoid_f(float z) { return fminf(z, 0.f) - log1pf(expf(-fabsf(z))); }
__device__ __forceinline__ float softplus_f(float z) { return fmaxf(z, 0.f) + log1pf(expf(-fabsf(z))); }

__device__ __forceinline__ float lanes_sum(float v) {
  v += __shfl_xor_sync(0xffffffffu, v, 1);
  v += __shfl_xor_sync(0xffffffffu, v, 2);
  v += __shfl_xor_sync(0xffffffffu, v, 4);
  return v;
}

// ---------------------------------------------------------------- matrix memory
// proj: float32 rows; q, k (heads x dim), v (heads x vdim) and the two gate projections (heads) start at the
// given columns.  state: per slot `state_stride` floats; per head [S: dim * vdim] and then, once for every
// kNormaliserColumns value columns, [n: dim][m: 1].  n and m do not depend on the column; every block keeps
// them for its own columns and reads and writes only the copies of its columns, so that no block reads what
// another block of the same launch has written.  R = rows of a lane, C = value columns of a block (a multiple
// of kNormaliserColumns).
template <int R, int C>
__global__ void __launch_bounds__(kLanes * C)
mlstm_scan_kernel(const float* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off, int i_off,
                  int f_off, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                  float q_scale, float* __restrict__ out, int out_stride, float* __restrict__ state,
                  long long state_stride, const int* __restrict__ query_start, const int* __restrict__ slots,
                  const int* __restrict__ request_active, int heads, int dim, int vdim, int max_slots, int* err) {
  constexpr int kPad = kLanes * R;
  __shared__ float k_s[2][kPad], q_s[2][kPad], gate_s[2][4];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int column = blockIdx.z * C + tid / kLanes, part = tid % kLanes;
  const bool live = column < vdim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  static_assert(C % kNormaliserColumns == 0, "a block owns whole copies of n and m");
  const int copies = (vdim + kNormaliserColumns - 1) / kNormaliserColumns;
  const int first_copy = blockIdx.z * (C / kNormaliserColumns);
  const int last_copy = min(first_copy + C / kNormaliserColumns, copies);
  float* s_base = state + (size_t)slot * state_stride + (size_t)head * ((size_t)dim * vdim + (size_t)copies * (dim + 1));
  float* n_base = s_base + (size_t)dim * vdim + (size_t)first_copy * (dim + 1);
  float s[R], n[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    s[i] = (live && row < dim) ? s_base[(size_t)row * vdim + column] : 0.f;
    n[i] = row < dim ? n_base[row] : 0.f;
  }
  float m = n_base[dim];
  for (int i = tid; i < 2 * kPad; i += blockDim.x) (&k_s[0][0])[i] = (&q_s[0][0])[i] = 0.f;
  __syncthreads();
  const float bi = i_bias[head], bf = f_bias[head];
  float kx = 0.f, qx = 0.f, ix = 0.f, fx = 0.f, vx = 0.f;
  auto fetch = [&](int t) {
    const float* row = proj + (size_t)t * proj_stride;
    if (tid < dim) {
      kx = row[k_off + head * dim + tid];
      qx = row[q_off + head * dim + tid];
    }
    if (tid == 0) {
      ix = row[i_off + head];
      fx = row[f_off + head];
    }
    if (live) vx = row[v_off + head * vdim + column];
  };
  if (begin < end) fetch(begin);
  for (int t = begin; t < end; ++t) {
    const int buf = (t - begin) & 1;
    if (tid < dim) {
      k_s[buf][tid] = kx;
      q_s[buf][tid] = qx * q_scale;
    }
    if (tid == 0) {
      const float gi = cap * tanhf((ix + bi) / cap);
      const float gf = log_sigmoid_f(cap * tanhf((fx + bf) / cap));
      const float m_new = fmaxf(gf + m, gi);
      gate_s[buf][0] = expf(gf + m - m_new);
      gate_s[buf][1] = expf(gi - m_new);
      gate_s[buf][2] = expf(-m_new);
      m = m_new;
    }
    const float v = vx;
    __syncthreads();
    if (t + 1 < end) fetch(t + 1);
    const float keep = gate_s[buf][0], take = gate_s[buf][1], floor_ = gate_s[buf][2];
    float o = 0.f, d = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      const float kk = take * k_s[buf][row], qq = q_s[buf][row];
      s[i] = fmaf(keep, s[i], kk * v);
      n[i] = fmaf(keep, n[i], kk);
      o = fmaf(qq, s[i], o);
      d = fmaf(qq, n[i], d);
    }
    o = lanes_sum(o);
    d = lanes_sum(d);
    if (live && part == 0) out[(size_t)t * out_stride + head * vdim + column] = o / (fmaxf(fabsf(d), floor_) + 1e-6f);
    // the buffers of token t are written again for token t + 2, after the barrier of token t + 1
  }
  if (!request_active[request]) return;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    if (row >= dim) continue;
    if (live) s_base[(size_t)row * vdim + column] = s[i];
    if (tid < kLanes)
      for (int copy = first_copy; copy < last_copy; ++copy) n_base[(size_t)(copy - first_copy) * (dim + 1) + row] = n[i];
  }
  if (tid == 0)
    for (int copy = first_copy; copy < last_copy; ++copy) n_base[(size_t)(copy - first_copy) * (dim + 1) + dim] = m;
}

// ---------------------------------------------------------------- short convolution + SiLU
// out[t][c] = silu(sum_j w[c][j] * x[t - (taps - 1 - j)][c]) over the channels c < channels of `proj` (its first
// columns), where x before the first token of this step comes from the request's history
// hist[(taps - 1)][channels] (oldest first) and is zero at the start of a request.  grid (tokens, channel blocks).
__global__ void short_conv_kernel(const float* __restrict__ proj, int proj_stride, const float* __restrict__ w,
                                  int taps, const float* __restrict__ state, long long state_stride,
                                  float* __restrict__ out, int out_stride, const int* __restrict__ query_start,
                                  const int* __restrict__ request_of_token, const int* __restrict__ slots,
                                  int channels, int max_slots, int* err) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int request = request_of_token[t];
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], place = t - begin;
  const float* hist = state + (size_t)slot * state_stride;
  float acc = 0.f;
  for (int j = 0; j < taps; ++j) {
    const int src = place - (taps - 1 - j);
    const float x = src >= 0 ? proj[(size_t)(begin + src) * proj_stride + c] : hist[(size_t)(taps - 1 + src) * channels + c];
    acc = fmaf(w[(size_t)c * taps + j], x, acc);
  }
  out[(size_t)t * out_stride + c] = acc / (1.f + expf(-acc));
}

// The history after this step: the inputs of the request's last taps - 1 tokens.  grid (requests, channel blocks).
__global__ void short_conv_keep_kernel(const float* __restrict__ proj, int proj_stride, int taps,
                                       float* __restrict__ state, long long state_stride,
                                       const int* __restrict__ query_start, const int* __restrict__ slots,
                                       const int* __restrict__ request_active, int channels, int max_slots) {
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, c = blockIdx.y * blockDim.x + threadIdx.x;
  if (c >= channels || !request_active[request]) return;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) return;
  const int begin = query_start[request], count = query_start[request + 1] - begin;
  float* hist = state + (size_t)slot * state_stride;
  float keep[kMaxTaps - 1];
#pragma unroll
  for (int j = 0; j < kMaxTaps - 1; ++j) {
    if (j >= taps - 1) break;
    const int src = count - (taps - 1) + j;
    keep[j] = src >= 0 ? proj[(size_t)(begin + src) * proj_stride + c] : hist[(size_t)(taps - 1 + src) * channels + c];
  }
#pragma unroll
  for (int j = 0; j < kMaxTaps - 1; ++j) {
    if (j >= taps - 1) break;
    hist[(size_t)j * channels + c] = keep[j];
  }
}

// ---------------------------------------------------------------- gated delta rule
// conv: float32 rows with q, k (kv_heads x dim) and v (heads x vdim) after convolution and SiLU at the given
// columns; proj: float32 rows with the write-strength and decay projections (heads each) at b_off, a_off.
// state: per slot `state_stride` floats; head h keeps S [dim][vdim] at h * dim * vdim.
template <int R, int C>
__global__ void __launch_bounds__(kLanes * C)
gated_delta_scan_kernel(const float* __restrict__ conv, int conv_stride, int q_off, int k_off, int v_off,
                        const float* __restrict__ proj, int proj_stride, int b_off, int a_off,
                        const float* __restrict__ a_log, const float* __restrict__ dt_bias, float q_scale,
                        float* __restrict__ out, int out_stride, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ query_start, const int* __restrict__ slots,
                        const int* __restrict__ request_active, int heads, int kv_heads, int dim, int vdim,
                        int max_slots, int* err) {
  constexpr int kPad = kLanes * R;
  __shared__ float k_s[2][kPad], q_s[2][kPad], gate_s[2][2];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int column = blockIdx.z * C + tid / kLanes, part = tid % kLanes;
  const bool live = column < vdim;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  const int shared_head = head / (heads / kv_heads);      // the q/k head this value head reads
  float* s_base = state + (size_t)slot * state_stride + (size_t)head * dim * vdim;
  float s[R];
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    s[i] = (live && row < dim) ? s_base[(size_t)row * vdim + column] : 0.f;
  }
  for (int i = tid; i < 2 * kPad; i += blockDim.x) (&k_s[0][0])[i] = (&q_s[0][0])[i] = 0.f;
  __syncthreads();
  const float rate = -expf(a_log[head]), dt = dt_bias[head];
  const bool stager = tid < ((dim + 31) / 32) * 32;     // whole warps whose threads own an element i = tid
  const int base = shared_head * dim;
  float kx = 0.f, qx = 0.f, ksq = 0.f, qsq = 0.f, bx = 0.f, ax = 0.f, vx = 0.f;
  auto fetch = [&](int t) {
    const float* row = conv + (size_t)t * conv_stride;
    if (stager) {
      ksq = qsq = 0.f;
      for (int i = lane; i < dim; i += 32) {       // every staging warp adds the same squares in the same order
        const float a = row[k_off + base + i], b = row[q_off + base + i];
        ksq = fmaf(a, a, ksq);
        qsq = fmaf(b, b, qsq);
      }
      if (tid < dim) {
        kx = row[k_off + base + tid];
        qx = row[q_off + base + tid];
      }
    }
    if (tid == 0) {
      bx = proj[(size_t)t * proj_stride + b_off + head];
      ax = proj[(size_t)t * proj_stride + a_off + head];
    }
    if (live) vx = row[v_off + head * vdim + column];
  };
  if (begin < end) fetch(begin);
  for (int t = begin; t < end; ++t) {
    const int buf = (t - begin) & 1;
    if (stager) {
      const float k_total = warp_sum(ksq), q_total = warp_sum(qsq);
      if (tid < dim) {
        k_s[buf][tid] = kx * rsqrtf(k_total + 1e-6f);
        q_s[buf][tid] = qx * rsqrtf(q_total + 1e-6f) * q_scale;
      }
    }
    if (tid == 0) {
      gate_s[buf][0] = expf(rate * softplus_f(ax + dt));
      gate_s[buf][1] = sigmoid_f(bx);
    }
    const float v = vx;
    __syncthreads();
    if (t + 1 < end) fetch(t + 1);
    const float g = gate_s[buf][0], beta = gate_s[buf][1];
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      s[i] *= g;
      dot = fmaf(k_s[buf][part * R + i], s[i], dot);
    }
    dot = lanes_sum(dot);
    const float u = beta * (v - dot);
    float o = 0.f;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int row = part * R + i;
      s[i] = fmaf(k_s[buf][row], u, s[i]);
      o = fmaf(q_s[buf][row], s[i], o);
    }
    o = lanes_sum(o);
    if (live && part == 0) out[(size_t)t * out_stride + head * vdim + column] = o;
  }
  if (!request_active[request] || !live) return;
#pragma unroll
  for (int i = 0; i < R; ++i) {
    const int row = part * R + i;
    if (row < dim) s_base[(size_t)row * vdim + column] = s[i];
  }
}

// ---------------------------------------------------------------- prompt portions: prepare, then stream
// For many tokens a request the scans above wait, token after token, for their own loads and for the
// exponentials of the gates.  Two kernels instead.  A prepare kernel works out, for all tokens at once, what
// the recurrence reads and packs it per head and token as float32 [k: P][q: P][gates: 4][v: VP] (k and q padded
// with zeros to P = 32, 64 or 128 rows, v to whole blocks of value columns).  Matrix memory: k, q * scale, the
// log input gate and the log forget gate.  Gated delta rule: the unit k, the unit q * scale, the decay and the
// write strength.  A stream kernel then walks a request's tokens with one thread (or two) a value column that
// keeps the rows of its column in registers, reading the packed rows through a ring of cp.async stages several
// tokens ahead: a shared-memory read is one address (or two neighbouring ones) for the whole warp.  The arithmetic
// is that of the scans; a column's sum over its rows is added as four chains.
//
// Matrix memory: the normaliser n is one more column whose value is 1 (n_t = keep n + take k * 1, and its
// read-out is n_t . q_t).  The first lane of one extra warp owns it; it writes max(|n . q|, exp(-m)) + 1e-6 per
// token and head, and the kernel that normalises the heads divides by it.  The running maximum is a chain of
// one addition and one maximum a token that every thread follows for itself.
constexpr int kStreamMaxDim = 128;    // largest key size: a column's rows are one thread's registers
constexpr int kStreamStages = 3;      // stages of the ring
constexpr int kStreamChunk = 4;       // tokens of a stage: the block meets once a stage, not once a token
constexpr int kStreamGates = 4;       // floats kept for the gates of a token (two used)
constexpr int kStreamColumns = 128;   // most value columns of a block

__host__ __device__ inline int stream_pad(int dim) { return dim <= 32 ? 32 : dim <= 64 ? 64 : 128; }
// Value columns of a block (a multiple of 32).  The matrix memory with 128 rows takes 64 at most: with its extra
// warp the block then has five warps, two a scheduler, and every thread may keep 255 registers.
__host__ __device__ inline int stream_block_columns(int dim, int vdim, bool memory) {
  const int limit = memory && stream_pad(dim) > 64 ? 64 : kStreamColumns;
  return vdim >= limit ? limit : (vdim + 31) / 32 * 32;
}
__host__ __device__ inline int stream_value_pad(int dim, int vdim, bool memory) {
  const int cb = stream_block_columns(dim, vdim, memory);
  return (vdim + cb - 1) / cb * cb;
}

// grid (tokens, heads)
__global__ void __launch_bounds__(128)
mlstm_prepare_kernel(const float* __restrict__ proj, int proj_stride, int q_off, int k_off, int v_off, int i_off,
                     int f_off, const float* __restrict__ i_bias, const float* __restrict__ f_bias, float cap,
                     float q_scale, float* __restrict__ packed, int tokens, int heads, int dim, int vdim) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int pad = stream_pad(dim), vpad = stream_value_pad(dim, vdim, true);
  const float* row = proj + (size_t)t * proj_stride;
  float* dst = packed + ((size_t)head * tokens + t) * (2 * pad + kStreamGates + vpad);
  for (int i = tid; i < pad; i += blockDim.x) {
    dst[i] = i < dim ? row[k_off + head * dim + i] : 0.f;
    dst[pad + i] = i < dim ? row[q_off + head * dim + i] * q_scale : 0.f;
  }
  if (tid < kStreamGates) {
    float g = 0.f;
    if (tid == 0) g = cap * tanhf((row[i_off + head] + i_bias[head]) / cap);
    if (tid == 1) g = log_sigmoid_f(cap * tanhf((row[f_off + head] + f_bias[head]) / cap));
    dst[2 * pad + tid] = g;
  }
  for (int i = tid; i < vpad; i += blockDim.x) dst[2 * pad + kStreamGates + i] = i < vdim ? row[v_off + head * vdim + i] : 0.f;
}

// grid (tokens, heads)
__global__ void __launch_bounds__(128)
gated_delta_prepare_kernel(const float* __restrict__ conv, int conv_stride, int q_off, int k_off, int v_off,
                           const float* __restrict__ proj, int proj_stride, int b_off, int a_off,
                           const float* __restrict__ a_log, const float* __restrict__ dt_bias, float q_scale,
                           float* __restrict__ packed, int tokens, int heads, int kv_heads, int dim, int vdim) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, head = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
  const int pad = stream_pad(dim), vpad = stream_value_pad(dim, vdim, false);
  const int base = (head / (heads / kv_heads)) * dim;
  const float* row = conv + (size_t)t * conv_stride;
  float ksq = 0.f, qsq = 0.f;
  for (int i = lane; i < dim; i += 32) {       // the order of the scan; every warp adds the same squares
    const float a = row[k_off + base + i], b = row[q_off + base + i];
    ksq = fmaf(a, a, ksq);
    qsq = fmaf(b, b, qsq);
  }
  const float k_inv = rsqrtf(warp_sum(ksq) + 1e-6f), q_inv = rsqrtf(warp_sum(qsq) + 1e-6f);
  float* dst = packed + ((size_t)head * tokens + t) * (2 * pad + kStreamGates + vpad);
  for (int i = tid; i < pad; i += blockDim.x) {
    dst[i] = i < dim ? row[k_off + base + i] * k_inv : 0.f;
    dst[pad + i] = i < dim ? row[q_off + base + i] * q_inv * q_scale : 0.f;
  }
  if (tid < kStreamGates) {
    float g = 0.f;
    if (tid == 0) g = expf(-expf(a_log[head]) * softplus_f(proj[(size_t)t * proj_stride + a_off + head] + dt_bias[head]));
    if (tid == 1) g = sigmoid_f(proj[(size_t)t * proj_stride + b_off + head]);
    dst[2 * pad + tid] = g;
  }
  for (int i = tid; i < vpad; i += blockDim.x) dst[2 * pad + kStreamGates + i] = i < vdim ? row[v_off + head * vdim + i] : 0.f;
}

__device__ __forceinline__ void stream_cp_async16(void* dst, const void* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src));
}

// grid (requests, heads, blocks of `cb` value columns, `cb` a multiple of 32); L threads a column, and one more
// warp for the matrix memory.  P = rows as padded; for P above 32 two neighbouring lanes share a column (L = 2):
// lane `part` keeps the rows of the 16-byte pieces part, part + L, ... of a token's k and q, so that the two read
// neighbouring pieces (no bank is asked twice), and one shuffle joins their sums.  kMemory: the matrix memory
// (state per head [S][copies x (n, m)] as the scan keeps it), else the gated delta rule (state per head [S]).
template <int L>
__device__ __forceinline__ float column_sum(float a, float b, float c, float d) {
  float x = (a + b) + (c + d);
  if (L == 2) x += __shfl_xor_sync(0xffffffffu, x, 1);
  return x;
}

template <int P, int L, bool kMemory>
__global__ void __launch_bounds__(kMemory ? (P > 64 ? 160 : L * kStreamColumns + 32) : L * kStreamColumns)
recurrent_stream_kernel(const float* __restrict__ packed, float* __restrict__ out, int out_stride,
                        float* __restrict__ denominators, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ query_start, const int* __restrict__ slots,
                        const int* __restrict__ request_active, int tokens, int heads, int dim, int vdim, int cb,
                        int max_slots, int* err) {
  constexpr int kHead = 2 * P + kStreamGates;          // k, q and gates of one token and head
  constexpr int kPieces = P / (4 * L);                 // 16-byte pieces of a row that a thread keeps
  __shared__ __align__(16) float ring[kStreamStages][kStreamChunk * (kHead + kStreamColumns)];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y, z = blockIdx.z, tid = threadIdx.x;
  const int local = tid / L, part = tid % L;
  const int column = z * cb + local;
  const bool live = local < cb && column < vdim;
  const bool normaliser = kMemory && local == cb;      // the column of n: the first L lanes of the extra warp
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  const int copies = (vdim + kNormaliserColumns - 1) / kNormaliserColumns;
  const int first_copy = z * (cb / kNormaliserColumns);
  const int last_copy = min(first_copy + cb / kNormaliserColumns, copies);
  const size_t head_floats = (size_t)dim * vdim + (kMemory ? (size_t)copies * (dim + 1) : 0);
  float* s_base = state + (size_t)slot * state_stride + (size_t)head * head_floats;
  float* n_base = s_base + (size_t)dim * vdim + (size_t)first_copy * (dim + 1);      // matrix memory only
  float s[4 * kPieces];                                // s[4 * i + j] is row 4 * (i * L + part) + j
#pragma unroll
  for (int i = 0; i < kPieces; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int row = 4 * (i * L + part) + j;
      float x = 0.f;
      if (row < dim) {
        if (live) x = s_base[(size_t)row * vdim + column];
        else if (normaliser) x = n_base[row];
      }
      s[4 * i + j] = x;
    }
  float m = kMemory ? n_base[dim] : 0.f;
  const int token_floats = kHead + cb;                 // floats of a token in the ring
  const int row_floats = kHead + stream_value_pad(dim, vdim, kMemory);
  const float* rows = packed + (size_t)head * tokens * row_floats;
  auto issue = [&](int chunk) {
    const int first = begin + chunk * kStreamChunk;
    if (first < end) {
      const int pieces = token_floats / 4, count = min(kStreamChunk, end - first) * pieces;
      float* dst = ring[chunk % kStreamStages];
      for (int c = tid; c < count; c += blockDim.x) {
        const int token = c / pieces, piece = c - token * pieces;
        const int from = 4 * piece < kHead ? 4 * piece : 4 * piece + z * cb;      // this block's value columns follow k, q, gates
        stream_cp_async16(dst + token * token_floats + 4 * piece, rows + (size_t)(first + token) * row_floats + from);
      }
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  for (int i = 0; i < kStreamStages - 1; ++i) issue(i);
  for (int t = begin; t < end; ++t) {
    const int chunk = (t - begin) / kStreamChunk, place = (t - begin) % kStreamChunk;
    if (place == 0) {
      asm volatile("cp.async.wait_group %0;\n" ::"n"(kStreamStages - 2));
      __syncthreads();          // the chunk has landed; everybody is done with the chunk before, whose stage is filled next
      issue(chunk + kStreamStages - 1);
    }
    const float* stage = ring[chunk % kStreamStages] + place * token_floats;
    const float4* k4 = reinterpret_cast<const float4*>(stage) + part;
    const float4* q4 = reinterpret_cast<const float4*>(stage + P) + part;
    const float gate0 = stage[2 * P], gate1 = stage[2 * P + 1];
    const float v = normaliser ? 1.f : stage[kHead + (local < cb ? local : 0)];
    float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;        // four chains, joined as (o0 + o1) + (o2 + o3)
    if (kMemory) {
      const float m_new = fmaxf(gate1 + m, gate0);
      const float keep = expf(gate1 + m - m_new), tv = expf(gate0 - m_new) * v;
      m = m_new;
#pragma unroll
      for (int i = 0; i < kPieces; ++i) {
        const float4 k = k4[i * L], q = q4[i * L];
        s[4 * i] = fmaf(keep, s[4 * i], k.x * tv);
        s[4 * i + 1] = fmaf(keep, s[4 * i + 1], k.y * tv);
        s[4 * i + 2] = fmaf(keep, s[4 * i + 2], k.z * tv);
        s[4 * i + 3] = fmaf(keep, s[4 * i + 3], k.w * tv);
        o0 = fmaf(q.x, s[4 * i], o0);
        o1 = fmaf(q.y, s[4 * i + 1], o1);
        o2 = fmaf(q.z, s[4 * i + 2], o2);
        o3 = fmaf(q.w, s[4 * i + 3], o3);
      }
      const float o = column_sum<L>(o0, o1, o2, o3);
      if (part == 0) {
        if (live) out[(size_t)t * out_stride + head * vdim + column] = o;
        if (normaliser && z == 0) denominators[(size_t)t * heads + head] = fmaxf(fabsf(o), expf(-m_new)) + 1e-6f;
      }
    } else {
      float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;
#pragma unroll
      for (int i = 0; i < kPieces; ++i) {
        const float4 k = k4[i * L];
        s[4 * i] *= gate0;
        s[4 * i + 1] *= gate0;
        s[4 * i + 2] *= gate0;
        s[4 * i + 3] *= gate0;
        d0 = fmaf(k.x, s[4 * i], d0);
        d1 = fmaf(k.y, s[4 * i + 1], d1);
        d2 = fmaf(k.z, s[4 * i + 2], d2);
        d3 = fmaf(k.w, s[4 * i + 3], d3);
      }
      const float u = gate1 * (v - column_sum<L>(d0, d1, d2, d3));
#pragma unroll
      for (int i = 0; i < kPieces; ++i) {
        const float4 k = k4[i * L], q = q4[i * L];
        s[4 * i] = fmaf(k.x, u, s[4 * i]);
        s[4 * i + 1] = fmaf(k.y, u, s[4 * i + 1]);
        s[4 * i + 2] = fmaf(k.z, u, s[4 * i + 2]);
        s[4 * i + 3] = fmaf(k.w, u, s[4 * i + 3]);
        o0 = fmaf(q.x, s[4 * i], o0);
        o1 = fmaf(q.y, s[4 * i + 1], o1);
        o2 = fmaf(q.z, s[4 * i + 2], o2);
        o3 = fmaf(q.w, s[4 * i + 3], o3);
      }
      const float o = column_sum<L>(o0, o1, o2, o3);
      if (live && part == 0) out[(size_t)t * out_stride + head * vdim + column] = o;
    }
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (!request_active[request]) return;
  if (live) {
#pragma unroll
    for (int i = 0; i < kPieces; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int row = 4 * (i * L + part) + j;
        if (row < dim) s_base[(size_t)row * vdim + column] = s[4 * i + j];
      }
  } else if (normaliser) {
    for (int copy = first_copy; copy < last_copy; ++copy) {
      float* to = n_base + (size_t)(copy - first_copy) * (dim + 1);
#pragma unroll
      for (int i = 0; i < kPieces; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const int row = 4 * (i * L + part) + j;
          if (row < dim) to[row] = s[4 * i + j];
        }
      if (part == 0) to[dim] = m;
    }
  }
}

// ---------------------------------------------------------------- per-head norm x gain x gate
// out[t][g*size + i] = gain * o / rms(o over the head) * act(gate); gain index i (shared) or g*size + i.  With
// `denominators` [tokens][heads], o is first divided by its token's and head's number.
// act 0: sigmoid(z), 1: z * sigmoid(z).  A warp per (token, head).
template <typename T>
__global__ void __launch_bounds__(32)
head_norm_gate_kernel(const float* __restrict__ o, int o_stride, const float* __restrict__ denominators,
                      const float* __restrict__ gate, int gate_stride, const float* __restrict__ gain, int gain_shared,
                      int act, T* __restrict__ out, int out_stride, int size, float eps) {
  pdl_wait();
  pdl_trigger();
  const int t = blockIdx.x, g = blockIdx.y, lane = threadIdx.x;
  const float* row = o + (size_t)t * o_stride + (size_t)g * size;
  const float below = denominators ? denominators[(size_t)t * gridDim.y + g] : 1.f;
  float sq = 0.f;
  for (int i = lane; i < size; i += 32) {
    const float x = row[i] / below;
    sq = fmaf(x, x, sq);
  }
  const float inv = rsqrtf(warp_sum(sq) / (float)size + eps);
  for (int i = lane; i < size; i += 32) {
    const int c = g * size + i;
    const float z = gate[(size_t)t * gate_stride + c];
    const float a = act ? z * sigmoid_f(z) : sigmoid_f(z);
    out[(size_t)t * out_stride + c] = from_float<T>(gain[gain_shared ? i : c] * ((row[i] / below) * inv) * a);
  }
}

}  // namespace cie

using namespace cie;

extern "C" int cie_scan_max_dim() { return kScanMaxDim; }
extern "C" int cie_conv_max_taps() { return kMaxTaps; }
extern "C" int cie_normaliser_columns() { return kNormaliserColumns; }

// Chooses the rows of a lane and the columns of a block from the sizes and runs BODY(R, C).
#define CIE_SCAN_SHAPES(name, dim, vdim, BODY)                                                           \
  do {                                                                                                   \
    if (dim < 1 || dim > kScanMaxDim || vdim < 1) CIE_FAIL("%s: head sizes %d / %d (keys up to %d)", name, dim, vdim, kScanMaxDim); \
    if (dim <= 32) { if (vdim <= 32) BODY(4, 32); else if (vdim <= 64) BODY(4, 64); else BODY(4, 128); }   \
    else if (dim <= 64) { if (vdim <= 32) BODY(8, 32); else if (vdim <= 64) BODY(8, 64); else BODY(8, 128); } \
    else if (dim <= 128) { if (vdim <= 32) BODY(16, 32); else if (vdim <= 64) BODY(16, 64); else BODY(16, 128); } \
    else { if (vdim <= 32) BODY(32, 32); else BODY(32, 64); }                                             \
  } while (0)

extern "C" int cie_mlstm_scan(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int i_off, int f_off,
                              const float* i_bias, const float* f_bias, float cap, float q_scale, float* out,
                              int out_stride, float* state, long long state_stride, const int* query_start,
                              const int* slots, const int* request_active, int requests, int heads, int dim,
                              int vdim, int max_slots, int* err, void* stream) {
  if (requests <= 0) return 0;
  if (heads < 1 || heads > 65535) CIE_FAIL("mlstm_scan: %d heads", heads);
  if (!(cap > 0.f)) CIE_FAIL("mlstm_scan: the gate cap must be positive, got %f", cap);
#define CIE_BODY(R, C)                                                                                          \
  CIE_LAUNCH("mlstm_scan", (mlstm_scan_kernel<R, C>), dim3(requests, heads, (vdim + C - 1) / C), dim3(kLanes * C), \
             0, (cudaStream_t)stream, proj, proj_stride, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, \
             q_scale, out, out_stride, state, state_stride, query_start, slots, request_active, heads, dim,      \
             vdim, max_slots, err)
  CIE_SCAN_SHAPES("mlstm_scan", dim, vdim, CIE_BODY);
#undef CIE_BODY
  return 0;
}

extern "C" int cie_gated_delta_scan(const float* conv, int conv_stride, int q_off, int k_off, int v_off,
                                    const float* proj, int proj_stride, int b_off, int a_off, const float* a_log,
                                    const float* dt_bias, float q_scale, float* out, int out_stride, float* state,
                                    long long state_stride, const int* query_start, const int* slots,
                                    const int* request_active, int requests, int heads, int kv_heads, int dim,
                                    int vdim, int max_slots, int* err, void* stream) {
  if (requests <= 0) return 0;
  if (heads < 1 || heads > 65535 || kv_heads < 1 || heads % kv_heads)
    CIE_FAIL("gated_delta_scan: %d heads do not divide over %d q/k heads", heads, kv_heads);
#define CIE_BODY(R, C)                                                                                          \
  CIE_LAUNCH("gated_delta_scan", (gated_delta_scan_kernel<R, C>), dim3(requests, heads, (vdim + C - 1) / C),      \
             dim3(kLanes * C), 0, (cudaStream_t)stream, conv, conv_stride, q_off, k_off, v_off, proj, proj_stride, \
             b_off, a_off, a_log, dt_bias, q_scale, out, out_stride, state, state_stride, query_start, slots,    \
             request_active, heads, kv_heads, dim, vdim, max_slots, err)
  CIE_SCAN_SHAPES("gated_delta_scan", dim, vdim, CIE_BODY);
#undef CIE_BODY
  return 0;
}

extern "C" int cie_stream_max_dim() { return kStreamMaxDim; }

// Floats of scratch memory the two-kernel form wants for `tokens` tokens.
extern "C" long long cie_recurrent_stream_floats(int tokens, int heads, int dim, int vdim, int memory) {
  return (long long)tokens * heads * (2 * stream_pad(dim) + kStreamGates + stream_value_pad(dim, vdim, memory != 0));
}

#define CIE_STREAM_LAUNCH(name, kMemory)                                                                          \
  do {                                                                                                            \
    const int cb = stream_block_columns(dim, vdim, kMemory), pad = stream_pad(dim), lanes = pad > 32 ? 2 : 1;                    \
    const dim3 grid(requests, heads, (vdim + cb - 1) / cb), block(lanes * cb + ((kMemory) ? 32 : 0));              \
    if (pad == 32)                                                                                                \
      CIE_LAUNCH(name, (recurrent_stream_kernel<32, 1, kMemory>), grid, block, 0, (cudaStream_t)stream, packed, out, \
                 out_stride, denominators, state, state_stride, query_start, slots, request_active, tokens, heads, \
                 dim, vdim, cb, max_slots, err);                                                                   \
    else if (pad == 64)                                                                                           \
      CIE_LAUNCH(name, (recurrent_stream_kernel<64, 2, kMemory>), grid, block, 0, (cudaStream_t)stream, packed, out, \
                 out_stride, denominators, state, state_stride, query_start, slots, request_active, tokens, heads, \
                 dim, vdim, cb, max_slots, err);                                                                   \
    else                                                                                                          \
      CIE_LAUNCH(name, (recurrent_stream_kernel<128, 2, kMemory>), grid, block, 0, (cudaStream_t)stream, packed, out, \
                 out_stride, denominators, state, state_stride, query_start, slots, request_active, tokens, heads, \
                 dim, vdim, cb, max_slots, err);                                                                   \
  } while (0)

// The matrix memory over prompt portions: `out` gets the numerators S_t^T q_t, `denominators` [tokens][heads]
// what they are to be divided by.
extern "C" int cie_mlstm_stream(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int i_off,
                                int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale,
                                float* packed, float* out, int out_stride, float* denominators, float* state,
                                long long state_stride, const int* query_start, const int* slots,
                                const int* request_active, int tokens, int requests, int heads, int dim, int vdim,
                                int max_slots, int* err, void* stream) {
  if (requests <= 0 || tokens <= 0) return 0;
  if (dim < 1 || dim > kStreamMaxDim || vdim < 1) CIE_FAIL("mlstm_stream: head sizes %d / %d (keys up to %d)", dim, vdim, kStreamMaxDim);
  if (heads < 1 || heads > 65535) CIE_FAIL("mlstm_stream: %d heads", heads);
  if (!(cap > 0.f)) CIE_FAIL("mlstm_stream: the gate cap must be positive, got %f", cap);
  CIE_LAUNCH("mlstm_prepare", mlstm_prepare_kernel, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream, proj,
             proj_stride, q_off, k_off, v_off, i_off, f_off, i_bias, f_bias, cap, q_scale, packed, tokens, heads, dim, vdim);
  CIE_STREAM_LAUNCH("mlstm_stream", true);
  return 0;
}

extern "C" int cie_gated_delta_stream(const float* conv, int conv_stride, int q_off, int k_off, int v_off,
                                      const float* proj, int proj_stride, int b_off, int a_off, const float* a_log,
                                      const float* dt_bias, float q_scale, float* packed, float* out, int out_stride,
                                      float* state, long long state_stride, const int* query_start, const int* slots,
                                      const int* request_active, int tokens, int requests, int heads, int kv_heads,
                                      int dim, int vdim, int max_slots, int* err, void* stream) {
  if (requests <= 0 || tokens <= 0) return 0;
  if (dim < 1 || dim > kStreamMaxDim || vdim < 1) CIE_FAIL("gated_delta_stream: head sizes %d / %d (keys up to %d)", dim, vdim, kStreamMaxDim);
  if (heads < 1 || heads > 65535 || kv_heads < 1 || heads % kv_heads)
    CIE_FAIL("gated_delta_stream: %d heads do not divide over %d q/k heads", heads, kv_heads);
  float* denominators = nullptr;
  CIE_LAUNCH("gated_delta_prepare", gated_delta_prepare_kernel, dim3(tokens, heads), dim3(128), 0, (cudaStream_t)stream,
             conv, conv_stride, q_off, k_off, v_off, proj, proj_stride, b_off, a_off, a_log, dt_bias, q_scale, packed,
             tokens, heads, kv_heads, dim, vdim);
  CIE_STREAM_LAUNCH("gated_delta_stream", false);
  return 0;
}

// The convolution of a step and then the history it leaves; `state` points at the history of slot 0.
extern "C" int cie_short_conv(const float* proj, int proj_stride, const float* w, int taps, float* state,
                              long long state_stride, float* out, int out_stride, const int* query_start,
                              const int* request_of_token, const int* slots, const int* request_active, int tokens,
                              int requests, int channels, int max_slots, int* err, void* stream) {
  if (tokens <= 0 || channels <= 0) return 0;
  if (taps < 1 || taps > kMaxTaps) CIE_FAIL("short_conv: %d taps (1..%d)", taps, kMaxTaps);
  const int threads = 256, blocks = (channels + threads - 1) / threads;
  CIE_LAUNCH("short_conv", short_conv_kernel, dim3(tokens, blocks), dim3(threads), 0, (cudaStream_t)stream, proj,
             proj_stride, w, taps, (const float*)state, state_stride, out, out_stride, query_start, request_of_token,
             slots, channels, max_slots, err);
  if (taps > 1)
    CIE_LAUNCH("short_conv_keep", short_conv_keep_kernel, dim3(requests, blocks), dim3(threads), 0,
               (cudaStream_t)stream, proj, proj_stride, taps, state, state_stride, query_start, slots, request_active,
               channels, max_slots);
  return 0;
}

extern "C" int cie_head_norm_gate(const float* o, int o_stride, const float* denominators, const float* gate, int gate_stride, const float* gain,
                                  int gain_shared, int act, void* out, int out_stride, int tokens, int groups,
                                  int size, float eps, int dtype, void* stream) {
  if (tokens <= 0 || groups <= 0) return 0;
  if (groups > 65535) CIE_FAIL("head_norm_gate: too many heads");
  if (act < 0 || act > 1) CIE_FAIL("head_norm_gate: unknown gate activation %d", act);
  if (dtype == kFloat32) {
    CIE_LAUNCH("head_norm_gate", head_norm_gate_kernel<float>, dim3(tokens, groups), dim3(32), 0, (cudaStream_t)stream,
               o, o_stride, denominators, gate, gate_stride, gain, gain_shared, act, (float*)out, out_stride, size, eps);
  } else if (dtype == kBFloat16) {
    CIE_LAUNCH("head_norm_gate", head_norm_gate_kernel<__nv_bfloat16>, dim3(tokens, groups), dim3(32), 0,
               (cudaStream_t)stream, o, o_stride, denominators, gate, gate_stride, gain, gain_shared, act, (__nv_bfloat16*)out,
               out_stride, size, eps);
  } else {
    CIE_FAIL("head_norm_gate: unknown dtype code %d", dtype);
  }
  return 0;
}
