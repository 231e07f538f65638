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
// tokens and state only, whatever the batch, the cut of a prompt into portions, or the slot (beyond the order of
// additions: prompt portions run in chunks of 32 tokens where the head sizes allow, else as a prepare kernel and
// a stream kernel with a thread a value column; the sections further down say how).
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
    if (tid == 2) g = -expf(a_log[head]) * softplus_f(proj[(size_t)t * proj_stride + a_off + head] + dt_bias[head]);   // log of the decay
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

// ---------------------------------------------------------------- matrix memory over prompt portions, in chunks
// The matrix memory's state is a sum over earlier tokens with weights that are products of scalars, so a
// prompt portion can be cut into chunks of kMemChunk tokens that many CTAs work on at once.  With b_t the log
// forget gates summed from the chunk's first token to t, m_t the running maximum (the recurrence above, taken
// token by token so that it is the same number in every form) and m_c the maximum before the chunk:
//   1. per token and head the two log gates; then per (request, head), one warp: b_t, m_t, m_(t-1)
//   2. per (chunk, head):               U = sum_s exp(b_last - b_s + i_s - m_last) k_s v_s^T, and the same with k_s alone
//   3. per (request, head):             walks its chunks, S <- exp(b_last + m_c - m_last) S + U, leaving in U's place
//                                       the state BEFORE the chunk; the last S, n and m go back to the slot
//   4. per (chunk, head):               o_t = (exp(b_t + m_c - m_t) S_c^T q_t + sum_(s<=t) a_ts v_s) / (max(|nq_t|, exp(-m_t)) + 1e-6),
//                                       a_ts = exp(b_t - b_s + i_s - m_t) (q_t . k_s),
//                                       nq_t = exp(b_t + m_c - m_t) (n_c . q_t) + sum_(s<=t) a_ts
// No exponent is above zero (m_t is at least every one of them), all float32 on the CUDA cores; key and value
// sizes up to kMemDim.  Chunks come as a work list made on the host; a request's chunks follow each other and
// start at multiples of kMemChunk tokens from the portion's first token.
constexpr int kMemChunk = 32;
constexpr int kMemWarps = 8;
constexpr int kMemDim = 128;                     // largest key and value size
constexpr int kMemRows = kMemDim / kMemWarps;    // state rows of a warp
constexpr int kMemCols = kMemDim / 32;           // value columns of a lane
constexpr int kMemGates = 4;                     // floats per token and head: i_t, b_t, m_t, m_(t-1)

// grid over tokens x heads: the two log gates of every token and head, left in the first two floats of its gates
__global__ void __launch_bounds__(256)
mlstm_gates_kernel(const float* __restrict__ proj, int proj_stride, int i_off, int f_off, const float* __restrict__ i_bias,
                   const float* __restrict__ f_bias, float cap, float* __restrict__ gates, int tokens, int heads) {
  pdl_wait();
  pdl_trigger();
  const int e = blockIdx.x * blockDim.x + threadIdx.x;
  if (e >= tokens * heads) return;
  const int t = e / heads, head = e % heads;
  const float* row = proj + (size_t)t * proj_stride;
  const float gi = cap * tanhf((row[i_off + head] + i_bias[head]) / cap);
  const float gf = log_sigmoid_f(cap * tanhf((row[f_off + head] + f_bias[head]) / cap));
  *reinterpret_cast<float2*>(gates + (size_t)e * kMemGates) = make_float2(gi, gf);
}

// grid (requests, heads); one warp.  The chain of a head is one addition and one maximum a token: the warp brings
// the gates of kWalkBlock tokens into shared memory, its first lane walks them there (the reads do not wait for the
// chain), and the warp carries the results out.
constexpr int kWalkBlock = 256;
__global__ void __launch_bounds__(32)
mlstm_gate_walk_kernel(const float* __restrict__ state, long long state_stride, float* __restrict__ gates,
                       const int* __restrict__ query_start, const int* __restrict__ slots, int heads, int dim, int vdim,
                       int max_slots, int* err) {
  static_assert(kWalkBlock % kMemChunk == 0, "a block of the walk holds whole chunks");
  __shared__ float2 in_s[kWalkBlock];
  __shared__ __align__(16) float4 out_s[kWalkBlock];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (lane == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int begin = query_start[request], end = query_start[request + 1];
  const int copies = (vdim + kNormaliserColumns - 1) / kNormaliserColumns;
  const size_t head_floats = (size_t)dim * vdim + (size_t)copies * (dim + 1);
  float m = state[(size_t)slot * state_stride + (size_t)head * head_floats + (size_t)dim * vdim + dim];
  float b = 0.f;
  for (int t0 = begin; t0 < end; t0 += kWalkBlock) {
    const int n = min(kWalkBlock, end - t0);
    for (int u = lane; u < n; u += 32)
      in_s[u] = *reinterpret_cast<const float2*>(gates + ((size_t)(t0 + u) * heads + head) * kMemGates);
    __syncwarp();
    if (lane == 0) {
#pragma unroll 8
      for (int u = 0; u < n; ++u) {
        const float2 g = in_s[u];
        b = u % kMemChunk == 0 ? g.y : b + g.y;
        const float m_new = fmaxf(g.y + m, g.x);
        out_s[u] = make_float4(g.x, b, m_new, m);
        m = m_new;
      }
    }
    __syncwarp();
    for (int u = lane; u < n; u += 32)
      *reinterpret_cast<float4*>(gates + ((size_t)(t0 + u) * heads + head) * kMemGates) = out_s[u];
    __syncwarp();
  }
}

// dst[j * ld + i] = proj[row0 + j][col0 + i] * factor(j) for j < n, i < width: 16-byte loads where the columns allow
template <typename Factor>
__device__ __forceinline__ void stage_rows(float* __restrict__ dst, int ld, const float* __restrict__ proj, int proj_stride,
                                           int row0, int n, int col0, int width, Factor factor) {
  if (width % 4 == 0 && col0 % 4 == 0 && proj_stride % 4 == 0 && ld % 4 == 0 && (reinterpret_cast<uintptr_t>(proj) & 15) == 0) {
    const int pieces = width / 4;
    for (int e = threadIdx.x; e < n * pieces; e += blockDim.x) {
      const int j = e / pieces, i = (e % pieces) * 4;
      float4 x = *reinterpret_cast<const float4*>(proj + (size_t)(row0 + j) * proj_stride + col0 + i);
      const float f = factor(j);
      x.x *= f; x.y *= f; x.z *= f; x.w *= f;
      *reinterpret_cast<float4*>(dst + j * ld + i) = x;
    }
    return;
  }
  for (int e = threadIdx.x; e < n * width; e += blockDim.x) {
    const int j = e / width, i = e % width;
    dst[j * ld + i] = proj[(size_t)(row0 + j) * proj_stride + col0 + i] * factor(j);
  }
}

// grid (chunks, heads).  chunk_sums: per chunk and head [U: dim * vdim][the same with k alone: dim]
__global__ void __launch_bounds__(kMemWarps * 32)
mlstm_chunk_sums_kernel(const float* __restrict__ proj, int proj_stride, int k_off, int v_off,
                        const float* __restrict__ gates, float* __restrict__ chunk_sums,
                        const int* __restrict__ chunk_row, const int* __restrict__ chunk_count, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  float* k_s = smem;                        // [kMemChunk][dim], times the token's weight
  float* v_s = smem + kMemChunk * dim;      // [kMemChunk][vdim]
  __shared__ float w_s[kMemChunk];
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  if (threadIdx.x < n) {
    const float4 g = *reinterpret_cast<const float4*>(gates + ((size_t)(row0 + threadIdx.x) * heads + head) * kMemGates);
    const float4 last = *reinterpret_cast<const float4*>(gates + ((size_t)(row0 + n - 1) * heads + head) * kMemGates);
    w_s[threadIdx.x] = expf(last.y - g.y + g.x - last.z);
  }
  __syncthreads();
  stage_rows(k_s, dim, proj, proj_stride, row0, n, k_off + head * dim, dim, [&](int j) { return w_s[j]; });
  stage_rows(v_s, vdim, proj, proj_stride, row0, n, v_off + head * vdim, vdim, [](int) { return 1.f; });
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int i0 = warp * kMemRows;
  const bool whole = dim % 4 == 0 && i0 + kMemRows <= dim;
  float u[kMemRows][kMemCols] = {};
  for (int j = 0; j < n; ++j) {
    float vv[kMemCols], kv[kMemRows];
#pragma unroll
    for (int c = 0; c < kMemCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
    if (whole) {
#pragma unroll
      for (int r = 0; r < kMemRows; r += 4) {
        const float4 k4 = *reinterpret_cast<const float4*>(k_s + j * dim + i0 + r);
        kv[r] = k4.x; kv[r + 1] = k4.y; kv[r + 2] = k4.z; kv[r + 3] = k4.w;
      }
    } else {
#pragma unroll
      for (int r = 0; r < kMemRows; ++r) kv[r] = i0 + r < dim ? k_s[j * dim + i0 + r] : 0.f;
    }
#pragma unroll
    for (int r = 0; r < kMemRows; ++r)
#pragma unroll
      for (int c = 0; c < kMemCols; ++c) u[r][c] = fmaf(kv[r], vv[c], u[r][c]);
  }
  float* dst = chunk_sums + ((size_t)chunk * heads + head) * ((size_t)dim * vdim + dim);
#pragma unroll
  for (int r = 0; r < kMemRows; ++r) {
    const int i = i0 + r;
    if (i >= dim) continue;
#pragma unroll
    for (int c = 0; c < kMemCols; ++c)
      if (lane + 32 * c < vdim) dst[(size_t)i * vdim + lane + 32 * c] = u[r][c];
  }
  for (int i = threadIdx.x; i < dim; i += blockDim.x) {
    float total = 0.f;
    for (int j = 0; j < n; ++j) total += k_s[j * dim + i];
    dst[(size_t)dim * vdim + i] = total;
  }
}

// grid (requests, heads, blocks over dim * vdim + dim + 1 cells: the matrix, the normaliser, the maximum)
__global__ void __launch_bounds__(256)
mlstm_chunk_prefix_kernel(float* __restrict__ chunk_sums, float* __restrict__ state, long long state_stride,
                          const float* __restrict__ gates, const int* __restrict__ request_chunk_start,
                          const int* __restrict__ chunk_row, const int* __restrict__ chunk_count,
                          const int* __restrict__ slots, const int* __restrict__ request_active, int heads, int dim,
                          int vdim, int max_slots, int* err) {
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y;
  const int e = blockIdx.z * blockDim.x + threadIdx.x;
  const int matrix = dim * vdim, cells = matrix + dim;
  if (e > cells) return;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (e == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const int copies = (vdim + kNormaliserColumns - 1) / kNormaliserColumns;
  const size_t head_floats = (size_t)matrix + (size_t)copies * (dim + 1);
  float* base = state + (size_t)slot * state_stride + (size_t)head * head_floats;
  const int first = request_chunk_start[request], last = request_chunk_start[request + 1];
  const bool active = request_active[request] != 0;
  if (e == cells) {                 // the running maximum after the request's last token
    if (active && last > first) {
      const int t = chunk_row[last - 1] + chunk_count[last - 1] - 1;
      const float m = gates[((size_t)t * heads + head) * kMemGates + 2];
      for (int copy = 0; copy < copies; ++copy) base[(size_t)matrix + (size_t)copy * (dim + 1) + dim] = m;
    }
    return;
  }
  float s = e < matrix ? base[e] : base[(size_t)matrix + (e - matrix)];
  const size_t stride = (size_t)heads * cells;
  constexpr int kBatch = 8;         // the sums of eight chunks are asked for together, before the first store
  for (int chunk = first; chunk < last; chunk += kBatch) {
    float* u = chunk_sums + ((size_t)chunk * heads + head) * cells + e;
    float gained[kBatch], power[kBatch];
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      const bool in = chunk + b < last;
      gained[b] = in ? u[b * stride] : 0.f;
      power[b] = 1.f;
      if (in) {
        const int tf = chunk_row[chunk + b], tl = tf + chunk_count[chunk + b] - 1;
        const float* gl = gates + ((size_t)tl * heads + head) * kMemGates;
        power[b] = expf(gl[1] + gates[((size_t)tf * heads + head) * kMemGates + 3] - gl[2]);
      }
    }
#pragma unroll
    for (int b = 0; b < kBatch; ++b) {
      if (chunk + b < last) {
        u[b * stride] = s;
        s = fmaf(power[b], s, gained[b]);
      }
    }
  }
  if (!active) return;
  if (e < matrix) base[e] = s;
  else
    for (int copy = 0; copy < copies; ++copy) base[(size_t)matrix + (size_t)copy * (dim + 1) + (e - matrix)] = s;
}

// grid (chunks, heads).  chunk_sums holds, after the walk, the state before each chunk.
// kMemory: the matrix memory (a denominator from the normaliser); else the gated delta rule in chunks (below), whose
// rows come with i_t = m_t = 0, b_t = the log decays summed from the chunk's first token, and v = the chunk's writes.
// q, k, v: where a head's rows are (see RowsOf).
struct RowsOf {
  const float* base;      // row t of head h starts at base + h * head_base + t * stride + col0 + h * head_col
  long long head_base;
  int stride, col0, head_col;
};

template <bool kMemory>
__global__ void __launch_bounds__(kMemWarps * 32)
chunk_output_kernel(RowsOf q_rows, RowsOf k_rows, RowsOf v_rows, float q_scale,
                    const float* __restrict__ gates, const float* __restrict__ chunk_sums,
                    float* __restrict__ out, int out_stride, const int* __restrict__ chunk_row,
                    const int* __restrict__ chunk_count, int heads, int dim, int vdim) {
  extern __shared__ __align__(16) float smem[];
  const int kd = dim + 1;                         // k rows are padded by one element: lanes run over keys
  float* q_s = smem;                              // [kMemChunk][dim]
  float* v_s = q_s + kMemChunk * dim;             // [kMemChunk][vdim]
  float* a_s = v_s + kMemChunk * vdim;            // [kMemChunk][kMemChunk]
  float* k_s = a_s + kMemChunk * kMemChunk;       // [kMemChunk][dim + 1]
  __shared__ float gi_s[kMemChunk], gb_s[kMemChunk], gm_s[kMemChunk];
  __shared__ float m_before;
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  if (threadIdx.x < n) {
    const float4 g = *reinterpret_cast<const float4*>(gates + ((size_t)(row0 + threadIdx.x) * heads + head) * kMemGates);
    gi_s[threadIdx.x] = g.x;
    gb_s[threadIdx.x] = g.y;
    gm_s[threadIdx.x] = g.z;
    if (threadIdx.x == 0) m_before = g.w;
  }
  stage_rows(q_s, dim, q_rows.base + head * q_rows.head_base, q_rows.stride, row0, n, q_rows.col0 + head * q_rows.head_col,
             dim, [&](int) { return q_scale; });
  stage_rows(k_s, kd, k_rows.base + head * k_rows.head_base, k_rows.stride, row0, n, k_rows.col0 + head * k_rows.head_col,
             dim, [](int) { return 1.f; });
  stage_rows(v_s, vdim, v_rows.base + head * v_rows.head_base, v_rows.stride, row0, n, v_rows.col0 + head * v_rows.head_col,
             vdim, [](int) { return 1.f; });
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  {
    // a warp takes four tokens that follow each other, a lane a key: a key's numbers are read once for four products
    constexpr int kQ = kMemChunk / kMemWarps;
    const int i0 = warp * kQ, j = lane;
    float dot[kQ] = {};
    if (i0 < n && j < n && j < i0 + kQ) {
      const int whole = dim % 4 == 0 ? dim : 0;
      for (int x = 0; x < whole; x += 4) {
        const float k0 = k_s[j * kd + x], k1 = k_s[j * kd + x + 1], k2 = k_s[j * kd + x + 2], k3 = k_s[j * kd + x + 3];
#pragma unroll
        for (int t = 0; t < kQ; ++t) {
          if (i0 + t >= n) break;
          const float4 q4 = *reinterpret_cast<const float4*>(q_s + (i0 + t) * dim + x);
          dot[t] = fmaf(q4.x, k0, dot[t]);
          dot[t] = fmaf(q4.y, k1, dot[t]);
          dot[t] = fmaf(q4.z, k2, dot[t]);
          dot[t] = fmaf(q4.w, k3, dot[t]);
        }
      }
      for (int x = whole; x < dim; ++x) {
        const float kx = k_s[j * kd + x];
#pragma unroll
        for (int t = 0; t < kQ; ++t)
          if (i0 + t < n) dot[t] = fmaf(q_s[(i0 + t) * dim + x], kx, dot[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < kQ; ++t) {
      const int i = i0 + t;
      a_s[i * kMemChunk + j] = (i < n && j <= i) ? dot[t] * expf(gb_s[i] - gb_s[j] + gi_s[j] - gm_s[i]) : 0.f;
    }
  }
  __syncthreads();
  const size_t cells = (size_t)dim * vdim + (kMemory ? dim : 0);
  const float* before = chunk_sums + ((size_t)chunk * heads + head) * cells;
  const float* n_before = before + (size_t)dim * vdim;
  // a warp takes tokens warp, warp + 8, ...; a lane the value columns lane, lane + 32, ...
  constexpr int kTokens = kMemChunk / kMemWarps;
  float carried[kTokens], below[kTokens];
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const int i = warp + kMemWarps * t;
    carried[t] = 0.f;
    below[t] = 1.f;
    if (i >= n) continue;
    carried[t] = expf(gb_s[i] + m_before - gm_s[i]);
    if (!kMemory) continue;
    float nq = 0.f;
    for (int x = lane; x < dim; x += 32) nq = fmaf(n_before[x], q_s[i * dim + x], nq);
    nq = warp_sum(nq) * carried[t] + warp_sum(lane <= i ? a_s[i * kMemChunk + lane] : 0.f);
    below[t] = fmaxf(fabsf(nq), expf(-gm_s[i])) + 1e-6f;
  }
  float inter[kTokens][kMemCols] = {}, intra[kTokens][kMemCols] = {};
  const int dim4 = dim % 4 == 0 ? dim : 0;       // four state rows a step where the q rows allow 16-byte loads
  for (int x = 0; x < dim4; x += 4) {
    float sv[4][kMemCols];
#pragma unroll
    for (int y = 0; y < 4; ++y)
#pragma unroll
      for (int c = 0; c < kMemCols; ++c) sv[y][c] = lane + 32 * c < vdim ? before[(size_t)(x + y) * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kMemWarps * t;
      const float4 q4 = i < n ? *reinterpret_cast<const float4*>(q_s + i * dim + x) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int c = 0; c < kMemCols; ++c) {
        inter[t][c] = fmaf(q4.x, sv[0][c], inter[t][c]);
        inter[t][c] = fmaf(q4.y, sv[1][c], inter[t][c]);
        inter[t][c] = fmaf(q4.z, sv[2][c], inter[t][c]);
        inter[t][c] = fmaf(q4.w, sv[3][c], inter[t][c]);
      }
    }
  }
  for (int x = dim4; x < dim; ++x) {
    float sv[kMemCols];
#pragma unroll
    for (int c = 0; c < kMemCols; ++c) sv[c] = lane + 32 * c < vdim ? before[(size_t)x * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kMemWarps * t;
      const float qv = i < n ? q_s[i * dim + x] : 0.f;
#pragma unroll
      for (int c = 0; c < kMemCols; ++c) inter[t][c] = fmaf(qv, sv[c], inter[t][c]);
    }
  }
  for (int j = 0; j < n; ++j) {
    float vv[kMemCols];
#pragma unroll
    for (int c = 0; c < kMemCols; ++c) vv[c] = lane + 32 * c < vdim ? v_s[j * vdim + lane + 32 * c] : 0.f;
#pragma unroll
    for (int t = 0; t < kTokens; ++t) {
      const int i = warp + kMemWarps * t;
      const float av = (i < n && j <= i) ? a_s[i * kMemChunk + j] : 0.f;
#pragma unroll
      for (int c = 0; c < kMemCols; ++c) intra[t][c] = fmaf(av, vv[c], intra[t][c]);
    }
  }
#pragma unroll
  for (int t = 0; t < kTokens; ++t) {
    const int i = warp + kMemWarps * t;
    if (i >= n) continue;
#pragma unroll
    for (int c = 0; c < kMemCols; ++c)
      if (lane + 32 * c < vdim)
        out[(size_t)(row0 + i) * out_stride + head * vdim + lane + 32 * c] = fmaf(carried[t], inter[t][c], intra[t][c]) / below[t];
  }
}

// ---------------------------------------------------------------- gated delta rule over prompt portions, in chunks
// Within a chunk of tokens 1..C that starts from the state S_0, with c_t the decays multiplied from the chunk's first
// token to t, the rule's writes u_t obey  u_t = b_t (v_t - c_t S_0^T k_t - sum_(s<t) (c_t / c_s) (k_s . k_t) u_s),  a
// triangular system:  (I + A) U = diag(b) (V - diag(c) K S_0),  A_ts = b_t (c_t / c_s) (k_t . k_s) for s < t.  With
// T = (I + A)^-1:  U = T diag(b) V - (T diag(b c) K) S_0 = U' - W S_0.  So:
//   1. prepare (above): unit k and q, decay, write strength and log decay of every token
//   2. per (chunk, head):      A, T by forward substitution (a lane a column of T), U' and W
//   3. per (request, head, 32 value columns): walks the chunks with its columns of S in registers:
//                              U = U' - W S_0,  S <- c_C S_0 + sum_s (c_C / c_s) k_s u_s^T; leaves S_0 of every chunk
//   4. per (chunk, head):      o_t = c_t S_0^T q_t + sum_(s<=t) (c_t / c_s) (q_t . k_s) u_s   (the matrix memory's output
//                              kernel with i = m = 0 and no denominator)
// Ratios of decays are exponentials of differences of summed logarithms, never quotients.  Float32 on the CUDA cores.
// Keys up to kMemDim, values a multiple of 4.
constexpr int kWalkColumns = 32;
constexpr int kWalkWarps = 16;                   // warps of the walk
constexpr int kWalkRows = kMemDim / kWalkWarps;  // state rows of a warp

// grid (chunks, heads).  packed: the prepared rows [k: P][q: P][gates][v: VP] per head and token.
__global__ void __launch_bounds__(256)
delta_chunk_solve_kernel(const float* __restrict__ packed, int tokens, int row_floats, int P,
                         float* __restrict__ gates, float* __restrict__ w_out, float* __restrict__ u_out,
                         const int* __restrict__ chunk_row, const int* __restrict__ chunk_count, int heads, int vdim) {
  constexpr int C = kMemChunk;
  extern __shared__ __align__(16) float smem[];
  const int kd = P + 1;
  float* v_s = smem;                       // [C][vdim]
  float* k_s = v_s + C * vdim;             // [C][P + 1]
  float* a_s = k_s + C * kd;               // [C][C + 1]
  float* t_s = a_s + C * (C + 1);          // [C][C + 1]
  __shared__ float beta_s[C], lg_s[C], bc_s[C];
  pdl_wait();
  pdl_trigger();
  const int chunk = blockIdx.x, head = blockIdx.y, tid = threadIdx.x;
  const int row0 = chunk_row[chunk], n = chunk_count[chunk];
  const float* rows = packed + (size_t)head * tokens * row_floats;
  if (tid < n) {
    float lg = 0.f;
    for (int r = 0; r <= tid; ++r) lg += rows[(size_t)(row0 + r) * row_floats + 2 * P + 2];
    const float beta = rows[(size_t)(row0 + tid) * row_floats + 2 * P + 1];
    lg_s[tid] = lg;
    beta_s[tid] = beta;
    bc_s[tid] = beta * expf(lg);
    *reinterpret_cast<float4*>(gates + ((size_t)(row0 + tid) * heads + head) * kMemGates) = make_float4(0.f, lg, 0.f, 0.f);
  }
  stage_rows(k_s, kd, rows, row_floats, row0, n, 0, P, [](int) { return 1.f; });
  stage_rows(v_s, vdim, rows, row_floats, row0, n, 2 * P + kStreamGates, vdim, [](int) { return 1.f; });
  __syncthreads();
  {
    // a warp takes four tokens that follow each other, a lane an earlier token
    constexpr int kQ = C / 8;
    const int t0 = (tid >> 5) * kQ, j = tid & 31;
    float a[kQ] = {};
    if (t0 < n && j < t0 + kQ - 1 && j < n) {
      for (int x = 0; x < P; ++x) {
        const float kx = k_s[j * kd + x];
#pragma unroll
        for (int t = 0; t < kQ; ++t) a[t] = fmaf(k_s[(t0 + t) * kd + x], kx, a[t]);
      }
    }
#pragma unroll
    for (int t = 0; t < kQ; ++t) {
      const int row = t0 + t;
      a_s[row * (C + 1) + j] = (j < row && row < n) ? a[t] * beta_s[row] * expf(lg_s[row] - lg_s[j]) : 0.f;
    }
  }
  __syncthreads();
  if (tid < C) {            // column tid of T = (I + A)^-1: T_tj = [t = j] - sum_(s<t) A_ts T_sj
    float col[C];
#pragma unroll
    for (int t = 0; t < C; ++t) {
      float x = t == tid ? 1.f : 0.f;
#pragma unroll
      for (int j = 0; j < t; ++j) x = fmaf(-a_s[t * (C + 1) + j], col[j], x);
      col[t] = x;
      t_s[t * (C + 1) + tid] = x;
    }
  }
  __syncthreads();
  const int wide = vdim + P;
  for (int e = tid; e < n * wide; e += blockDim.x) {
    const int t = e / wide, c = e % wide;
    float acc = 0.f;
    if (c < vdim) {
      for (int j = 0; j <= t; ++j) acc = fmaf(t_s[t * (C + 1) + j] * beta_s[j], v_s[j * vdim + c], acc);
      u_out[((size_t)(row0 + t) * heads + head) * vdim + c] = acc;
    } else {
      const int x = c - vdim;
      for (int j = 0; j <= t; ++j) acc = fmaf(t_s[t * (C + 1) + j] * bc_s[j], k_s[j * kd + x], acc);
      w_out[((size_t)(row0 + t) * heads + head) * P + x] = acc;
    }
  }
}

// grid (requests, heads, blocks of kWalkColumns value columns); warp w keeps kWalkRows state rows of the block's
// columns in registers, a lane a column.  What a chunk brings (W, k, U', the summed log decays) comes
// through two cp.async stages, a chunk ahead.
__global__ void __launch_bounds__(kWalkWarps * 32)
delta_chunk_walk_kernel(const float* __restrict__ packed, int tokens, int row_floats, int P,
                        const float* __restrict__ gates, const float* __restrict__ w_in, float* __restrict__ u_io,
                        float* __restrict__ before, float* __restrict__ state, long long state_stride,
                        const int* __restrict__ request_chunk_start, const int* __restrict__ chunk_row,
                        const int* __restrict__ chunk_count, const int* __restrict__ slots,
                        const int* __restrict__ request_active, int heads, int dim, int vdim, int max_slots, int* err) {
  constexpr int C = kMemChunk, kRows = kWalkRows, kCols = kWalkColumns;
  extern __shared__ __align__(16) float smem[];
  const int stage_floats = 2 * C * P + C * kCols + C * kMemGates;
  float* part_s = smem + 2 * stage_floats;        // [warps][C][kCols]
  float* u_s = part_s + kWalkWarps * C * kCols;   // [C][kCols]
  __shared__ float weight_s[C];
  pdl_wait();
  pdl_trigger();
  const int request = blockIdx.x, head = blockIdx.y, col0 = blockIdx.z * kCols, tid = threadIdx.x;
  const int warp = tid >> 5, lane = tid & 31, column = col0 + lane, r0 = warp * kRows;
  const int slot = slots[request];
  if (slot < 0 || slot >= max_slots) {
    if (tid == 0) atomicOr(err, kErrBadRequest);
    return;
  }
  const bool live = column < vdim;
  const int warps = P / kRows;                     // warps that hold rows
  float* s_base = state + (size_t)slot * state_stride + (size_t)head * dim * vdim;
  float s[kRows];
#pragma unroll
  for (int r = 0; r < kRows; ++r) s[r] = (live && r0 + r < dim) ? s_base[(size_t)(r0 + r) * vdim + column] : 0.f;
  const int first = request_chunk_start[request], last = request_chunk_start[request + 1];
  const float* rows = packed + (size_t)head * tokens * row_floats;
  const int columns = min(kCols, vdim - col0);     // a multiple of 4, as vdim is
  auto issue = [&](int chunk) {
    if (chunk < last) {
      float* dst = smem + (size_t)((chunk - first) & 1) * stage_floats;
      const int row0 = chunk_row[chunk], n = chunk_count[chunk];
      const int pw = P / 4, pu = columns / 4;
      for (int c = tid; c < n * pw; c += blockDim.x) {
        const int t = c / pw, piece = c % pw;
        stream_cp_async16(dst + t * P + 4 * piece, w_in + ((size_t)(row0 + t) * heads + head) * P + 4 * piece);
        stream_cp_async16(dst + C * P + t * P + 4 * piece, rows + (size_t)(row0 + t) * row_floats + 4 * piece);
      }
      for (int c = tid; c < n * pu; c += blockDim.x) {
        const int t = c / pu, piece = c % pu;
        stream_cp_async16(dst + 2 * C * P + t * kCols + 4 * piece,
                          u_io + ((size_t)(row0 + t) * heads + head) * vdim + col0 + 4 * piece);
      }
      for (int t = tid; t < n; t += blockDim.x)
        stream_cp_async16(dst + 2 * C * P + C * kCols + t * kMemGates, gates + ((size_t)(row0 + t) * heads + head) * kMemGates);
    }
    asm volatile("cp.async.commit_group;\n" ::);
  };
  issue(first);
  for (int chunk = first; chunk < last; ++chunk) {
    const float* w_s = smem + (size_t)((chunk - first) & 1) * stage_floats;
    const float* k_s = w_s + C * P;
    const float* ut_s = k_s + C * P;
    const float* g_s = ut_s + C * kCols;
    const int row0 = chunk_row[chunk], n = chunk_count[chunk];
    issue(chunk + 1);
    asm volatile("cp.async.wait_group 1;\n" ::);
    __syncthreads();
    if (warp < warps) {
      float* dst = before + ((size_t)chunk * heads + head) * dim * vdim;
#pragma unroll
      for (int r = 0; r < kRows; ++r)
        if (live && r0 + r < dim) dst[(size_t)(r0 + r) * vdim + column] = s[r];
      for (int t = 0; t < n; ++t) {
        float acc = 0.f;
#pragma unroll
        for (int r = 0; r < kRows; r += 4) {
          const float4 w4 = *reinterpret_cast<const float4*>(w_s + t * P + r0 + r);
          acc = fmaf(w4.x, s[r], acc);
          acc = fmaf(w4.y, s[r + 1], acc);
          acc = fmaf(w4.z, s[r + 2], acc);
          acc = fmaf(w4.w, s[r + 3], acc);
        }
        part_s[(warp * C + t) * kCols + lane] = acc;
      }
    }
    __syncthreads();
    if (tid < n) weight_s[tid] = expf(g_s[(n - 1) * kMemGates + 1] - g_s[tid * kMemGates + 1]);
    for (int t = warp; t < n; t += kWalkWarps) {
      float u = ut_s[t * kCols + lane];
      for (int w = 0; w < warps; ++w) u -= part_s[(w * C + t) * kCols + lane];
      u_s[t * kCols + lane] = u;
      if (live) u_io[((size_t)(row0 + t) * heads + head) * vdim + column] = u;
    }
    __syncthreads();
    if (warp < warps) {
      const float lg_last = g_s[(n - 1) * kMemGates + 1];
      const float keep = expf(lg_last);
#pragma unroll
      for (int r = 0; r < kRows; ++r) s[r] *= keep;
      for (int t = 0; t < n; ++t) {
        const float u = u_s[t * kCols + lane] * weight_s[t];
#pragma unroll
        for (int r = 0; r < kRows; r += 4) {
          const float4 k4 = *reinterpret_cast<const float4*>(k_s + t * P + r0 + r);
          s[r] = fmaf(k4.x, u, s[r]);
          s[r + 1] = fmaf(k4.y, u, s[r + 1]);
          s[r + 2] = fmaf(k4.z, u, s[r + 2]);
          s[r + 3] = fmaf(k4.w, u, s[r + 3]);
        }
      }
    }
    __syncthreads();        // everybody is done with this chunk's stage and with u_s before they are filled again
  }
  asm volatile("cp.async.wait_group 0;\n" ::);
  if (!request_active[request] || !live) return;
#pragma unroll
  for (int r = 0; r < kRows; ++r)
    if (r0 + r < dim) s_base[(size_t)(r0 + r) * vdim + column] = s[r];
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

extern "C" int cie_mlstm_chunk_tokens() { return kMemChunk; }
extern "C" int cie_mlstm_chunk_max_dim() { return kMemDim; }

// Floats of scratch memory the chunked form wants: every token's gates, then every chunk's sums.
extern "C" long long cie_mlstm_chunk_floats(int tokens, int chunks, int heads, int dim, int vdim) {
  return (long long)tokens * heads * kMemGates + (long long)chunks * heads * ((long long)dim * vdim + dim);
}

// The matrix memory over a step with prompt portions, in chunks (work lists from the host: first token row and
// token count of every chunk, and where every request's chunks start).  `out` gets the mixer's output.
extern "C" int cie_mlstm_chunked(const float* proj, int proj_stride, int q_off, int k_off, int v_off, int i_off,
                                 int f_off, const float* i_bias, const float* f_bias, float cap, float q_scale,
                                 float* scratch, float* out, int out_stride, float* state, long long state_stride,
                                 const int* query_start, const int* slots, const int* request_active,
                                 const int* chunk_row, const int* chunk_count, const int* request_chunk_start,
                                 int tokens, int chunks, int requests, int heads, int dim, int vdim, int max_slots,
                                 int* err, void* stream) {
  if (requests <= 0 || tokens <= 0 || chunks <= 0) return 0;
  if (dim < 1 || dim > kMemDim || vdim < 1 || vdim > kMemDim)
    CIE_FAIL("mlstm_chunked: key / value sizes %d / %d are outside 1..%d", dim, vdim, kMemDim);
  if (heads < 1 || heads > 65535) CIE_FAIL("mlstm_chunked: %d heads", heads);
  if (!(cap > 0.f)) CIE_FAIL("mlstm_chunked: the gate cap must be positive, got %f", cap);
  cudaStream_t s = (cudaStream_t)stream;
  float* gates = scratch;
  float* sums = scratch + (size_t)tokens * heads * kMemGates;
  const size_t smem2 = (size_t)kMemChunk * (dim + vdim) * sizeof(float);
  const size_t smem4 = (size_t)kMemChunk * (2 * dim + 1 + vdim + kMemChunk) * sizeof(float);
  if (smem4 > 48 * 1024 && cudaFuncSetAttribute(chunk_output_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                (int)smem4) != cudaSuccess)
    CIE_FAIL("mlstm_chunked: cannot reserve %zu bytes of shared memory", smem4);
  const dim3 grid(chunks, heads), block(kMemWarps * 32);
  CIE_LAUNCH("mlstm_gates", mlstm_gates_kernel, dim3((tokens * heads + 255) / 256), dim3(256), 0, s, proj, proj_stride,
             i_off, f_off, i_bias, f_bias, cap, gates, tokens, heads);
  CIE_LAUNCH("mlstm_gate_walk", mlstm_gate_walk_kernel, dim3(requests, heads), dim3(32), 0, s,
             (const float*)state, state_stride, gates, query_start, slots, heads, dim, vdim, max_slots, err);
  CIE_LAUNCH("mlstm_chunk_sums", mlstm_chunk_sums_kernel, grid, block, smem2, s, proj, proj_stride, k_off, v_off,
             (const float*)gates, sums, chunk_row, chunk_count, heads, dim, vdim);
  CIE_LAUNCH("mlstm_chunk_prefix", mlstm_chunk_prefix_kernel, dim3(requests, heads, (dim * vdim + dim + 1 + 255) / 256),
             dim3(256), 0, s, sums, state, state_stride, (const float*)gates, request_chunk_start, chunk_row, chunk_count,
             slots, request_active, heads, dim, vdim, max_slots, err);
  const RowsOf q_rows{proj, 0, proj_stride, q_off, dim}, k_rows{proj, 0, proj_stride, k_off, dim}, v_rows{proj, 0, proj_stride, v_off, vdim};
  CIE_LAUNCH("mlstm_chunk_output", chunk_output_kernel<true>, grid, block, smem4, s, q_rows, k_rows, v_rows, q_scale,
             (const float*)gates, (const float*)sums, out, out_stride, chunk_row, chunk_count, heads, dim, vdim);
  return 0;
}

// Floats of scratch memory the gated delta rule in chunks wants: the prepared rows, every token's summed log decays,
// W and U per token, and the state before every chunk.
extern "C" long long cie_gated_delta_chunk_floats(int tokens, int chunks, int heads, int dim, int vdim) {
  const long long row = 2 * stream_pad(dim) + kStreamGates + stream_value_pad(dim, vdim, false);
  return (long long)tokens * heads * (row + kMemGates + stream_pad(dim) + vdim) + (long long)chunks * heads * dim * vdim;
}

// The gated delta rule over a step with prompt portions, in chunks of cie_mlstm_chunk_tokens() tokens (work lists as
// for the matrix memory).  Keys up to cie_mlstm_chunk_max_dim(), values up to the same and a multiple of 4.
extern "C" int cie_gated_delta_chunked(const float* conv, int conv_stride, int q_off, int k_off, int v_off,
                                       const float* proj, int proj_stride, int b_off, int a_off, const float* a_log,
                                       const float* dt_bias, float q_scale, float* scratch, float* out, int out_stride,
                                       float* state, long long state_stride, const int* slots, const int* request_active,
                                       const int* chunk_row, const int* chunk_count, const int* request_chunk_start,
                                       int tokens, int chunks, int requests, int heads, int kv_heads, int dim, int vdim,
                                       int max_slots, int* err, void* stream) {
  if (requests <= 0 || tokens <= 0 || chunks <= 0) return 0;
  if (dim < 1 || dim > kMemDim || vdim < 4 || vdim > kMemDim || vdim % 4)
    CIE_FAIL("gated_delta_chunked: key / value sizes %d / %d (keys up to %d, values a multiple of 4 up to %d)", dim, vdim,
             kMemDim, kMemDim);
  if (heads < 1 || heads > 65535 || kv_heads < 1 || heads % kv_heads)
    CIE_FAIL("gated_delta_chunked: %d heads do not divide over %d q/k heads", heads, kv_heads);
  cudaStream_t s = (cudaStream_t)stream;
  const int P = stream_pad(dim), row_floats = 2 * P + kStreamGates + stream_value_pad(dim, vdim, false);
  float* packed = scratch;
  float* gates = packed + (size_t)tokens * heads * row_floats;
  float* w = gates + (size_t)tokens * heads * kMemGates;
  float* u = w + (size_t)tokens * heads * P;
  float* before = u + (size_t)tokens * heads * vdim;
  const size_t smem2 = (size_t)(kMemChunk * (vdim + P + 1) + 2 * kMemChunk * (kMemChunk + 1)) * sizeof(float);
  const size_t smem3 = (size_t)(2 * (2 * kMemChunk * P + kMemChunk * kWalkColumns + kMemChunk * kMemGates) +
                                (kWalkWarps + 1) * kMemChunk * kWalkColumns) * sizeof(float);
  const size_t smem4 = (size_t)kMemChunk * (2 * dim + 1 + vdim + kMemChunk) * sizeof(float);
  if (cudaFuncSetAttribute(delta_chunk_solve_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem2) != cudaSuccess ||
      cudaFuncSetAttribute(delta_chunk_walk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3) != cudaSuccess ||
      cudaFuncSetAttribute(chunk_output_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem4) != cudaSuccess)
    CIE_FAIL("gated_delta_chunked: cannot reserve %zu / %zu / %zu bytes of shared memory", smem2, smem3, smem4);
  CIE_LAUNCH("gated_delta_prepare", gated_delta_prepare_kernel, dim3(tokens, heads), dim3(128), 0, s, conv, conv_stride,
             q_off, k_off, v_off, proj, proj_stride, b_off, a_off, a_log, dt_bias, q_scale, packed, tokens, heads, kv_heads,
             dim, vdim);
  const dim3 grid(chunks, heads);
  CIE_LAUNCH("delta_chunk_solve", delta_chunk_solve_kernel, grid, dim3(256), smem2, s, (const float*)packed, tokens,
             row_floats, P, gates, w, u, chunk_row, chunk_count, heads, vdim);
  CIE_LAUNCH("delta_chunk_walk", delta_chunk_walk_kernel, dim3(requests, heads, (vdim + kWalkColumns - 1) / kWalkColumns),
             dim3(kWalkWarps * 32), smem3, s, (const float*)packed, tokens, row_floats, P, (const float*)gates, (const float*)w, u,
             before, state, state_stride, request_chunk_start, chunk_row, chunk_count, slots, request_active, heads, dim,
             vdim, max_slots, err);
  const RowsOf q_rows{packed, (long long)tokens * row_floats, row_floats, P, 0};
  const RowsOf k_rows{packed, (long long)tokens * row_floats, row_floats, 0, 0};
  const RowsOf v_rows{u, 0, heads * vdim, 0, vdim};
  CIE_LAUNCH("delta_chunk_output", chunk_output_kernel<false>, grid, dim3(kMemWarps * 32), smem4, s, q_rows, k_rows, v_rows,
             1.f, (const float*)gates, (const float*)before, out, out_stride, chunk_row, chunk_count, heads, dim, vdim);
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
