// Mixers whose memory is a matrix per head instead of a list of keys: S [dim, vdim] in float32 per (sequence, head),
// carried from token to token in the cache's fixed-size state.
//
//   decayed outer products:  S <- decay_h S + k_t v_t^T;                          o_t = S^T q_t
//   gated delta rule:        S <- g_t S;  u = beta_t (v_t - S^T k_t);  S <- S + k_t u^T;  o_t = S^T q_t
//
// One kernel serves prompts and single tokens: a block owns 16 columns of one head's S for one sequence and walks
// that sequence's new tokens in order, from the state the cache holds to the state it leaves there. A column's
// recurrence does not involve the other columns, so columns are the parallel dimension besides heads and sequences.
// Inside a warp a lane holds `RPL` consecutive rows of one column (8 lanes a column, 4 columns a warp): the sums over
// rows (S^T q, S^T k) are RPL multiply-adds a lane and three shuffles. The tokens' q, k and v come through two
// shared-memory stages filled by cp.async, so global latency is paid once per 16 tokens and hidden behind the
// arithmetic of the stage before. Everything is float32: inputs, state, sums.
//
// State layout: [slot][head][column][row], a column's rows contiguous (a lane's rows are one or more 16-byte loads).
#include "common.cuh"

#define SCAN_WARPS 4
#define SCAN_COLS (4 * SCAN_WARPS)
#define SCAN_THREADS (32 * SCAN_WARPS)

__device__ __forceinline__ void cp_async4(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(s), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ float silu_exact(float g) {
  float s;
  if (g >= 0.f) {
    s = 1.0f / (1.0f + expf(-g));
  } else {
    float e = expf(g);
    s = e / (1.0f + e);
  }
  return g * s;
}
__device__ __forceinline__ float sigmoid_exact(float g) {
  if (g >= 0.f) return 1.0f / (1.0f + expf(-g));
  float e = expf(g);
  return e / (1.0f + e);
}

struct ScanArgs {
  const float* q;        // rows of `stride` floats; a token's q of head j starts at q + token * stride + j * dim
  const float* k;
  const float* v;        // a token's v of head h starts at v + token * stride + h * vdim
  int stride;
  int heads, qk_heads;   // head h reads q/k head h / (heads / qk_heads)
  int dim, vdim;
  float* state;          // [slots][heads][vdim][dim]
  const int* cu_seqlens; // sequence s has the tokens cu_seqlens[s] .. cu_seqlens[s + 1] - 1 of the step
  const int* slots;
  float* out;            // [tokens][heads * vdim]
  // decayed outer products
  const float* decay;    // [heads]
  int activation;        // 1: q, k and v pass silu on the way in
  float k_scale;
  // gated delta rule: per token [g (heads) | beta (heads) | k.q (qk_heads)], `aux_stride` floats a token
  const float* aux;
  int aux_stride;
};

// MODE 0: decayed outer products; MODE 1: gated delta rule. TOKENS: tokens a stage.
template <int RPL, int MODE, int TOKENS>
__global__ void __launch_bounds__(SCAN_THREADS) scan_kernel(ScanArgs a) {
  constexpr int DIMP = RPL * 8;  // rows a stage holds per token (the head's dim rounded up)
  constexpr int PER_TOKEN = 2 * DIMP + SCAN_COLS + 4;
  extern __shared__ __align__(16) float stage[];  // [2][TOKENS][PER_TOKEN]: k | q | v (16 columns) | g, beta, k.q, -
  pdl_launch_dependents();
  const int head = blockIdx.y, seq = blockIdx.z, col0 = blockIdx.x * SCAN_COLS;
  const int qk_head = head / (a.heads / a.qk_heads);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int rg = lane >> 2, cc = lane & 3;
  const int col = col0 + warp * 4 + cc;
  const float decay = MODE == 0 ? a.decay[head] : 0.f;
  pdl_wait();
  const int first = a.cu_seqlens[seq], count = a.cu_seqlens[seq + 1] - first;
  const int slot = a.slots[seq];
  float* my_state = a.state + (((size_t)slot * a.heads + head) * a.vdim + col) * (size_t)a.dim + rg * RPL;

  float S[RPL];
#pragma unroll
  for (int j = 0; j < RPL; ++j) S[j] = (col < a.vdim && rg * RPL + j < a.dim) ? my_state[j] : 0.f;

  auto fill = [&](int chunk, int buffer) {
    float* dst = stage + (size_t)buffer * TOKENS * PER_TOKEN;
    int t0 = chunk * TOKENS;
    for (int i = tid; i < TOKENS * PER_TOKEN; i += SCAN_THREADS) {
      int t = i / PER_TOKEN, e = i - t * PER_TOKEN;
      const float* src = nullptr;
      if (t0 + t < count) {
        size_t token = (size_t)(first + t0 + t);
        if (e < DIMP) {
          if (e < a.dim) src = a.k + token * a.stride + qk_head * a.dim + e;
        } else if (e < 2 * DIMP) {
          if (e - DIMP < a.dim) src = a.q + token * a.stride + qk_head * a.dim + (e - DIMP);
        } else if (e < 2 * DIMP + SCAN_COLS) {
          int c = col0 + e - 2 * DIMP;
          if (c < a.vdim) src = a.v + token * a.stride + head * a.vdim + c;
        } else if (MODE == 1) {
          int which = e - 2 * DIMP - SCAN_COLS;
          if (which == 0) src = a.aux + token * a.aux_stride + head;
          else if (which == 1) src = a.aux + token * a.aux_stride + a.heads + head;
          else if (which == 2) src = a.aux + token * a.aux_stride + 2 * a.heads + qk_head;
        }
      }
      if (src != nullptr) cp_async4(dst + i, src);
      else dst[i] = 0.f;
    }
    cp_async_commit();
  };
  // what a thread copied it also finishes (the same index walk): activation or scale in place
  auto finish = [&](int buffer) {
    if (MODE != 0 || (a.activation == 0 && a.k_scale == 1.0f)) return;
    float* dst = stage + (size_t)buffer * TOKENS * PER_TOKEN;
    for (int i = tid; i < TOKENS * PER_TOKEN; i += SCAN_THREADS) {
      int e = i % PER_TOKEN;
      if (e >= 2 * DIMP + SCAN_COLS) continue;
      float value = dst[i];
      if (a.activation == 1) value = silu_exact(value);
      if (e < DIMP) value *= a.k_scale;
      dst[i] = value;
    }
  };

  const int chunks = (count + TOKENS - 1) / TOKENS;
  if (chunks > 0) fill(0, 0);
  for (int chunk = 0; chunk < chunks; ++chunk) {
    int buffer = chunk & 1;
    if (chunk + 1 < chunks) {
      fill(chunk + 1, buffer ^ 1);
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    finish(buffer);
    __syncthreads();
    const float* base = stage + (size_t)buffer * TOKENS * PER_TOKEN;
    int here = min(TOKENS, count - chunk * TOKENS);
    for (int t = 0; t < here; ++t) {
      const float* row = base + t * PER_TOKEN;
      float kk[RPL], qq[RPL];
#pragma unroll
      for (int j = 0; j < RPL; j += 4) {
        float4 k4 = *reinterpret_cast<const float4*>(row + rg * RPL + j);
        float4 q4 = *reinterpret_cast<const float4*>(row + DIMP + rg * RPL + j);
        kk[j] = k4.x; kk[j + 1] = k4.y; kk[j + 2] = k4.z; kk[j + 3] = k4.w;
        qq[j] = q4.x; qq[j + 1] = q4.y; qq[j + 2] = q4.z; qq[j + 3] = q4.w;
      }
      float v = row[2 * DIMP + warp * 4 + cc];
      float o;
      if (MODE == 0) {
        float p = 0.f;
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          S[j] = fmaf(decay, S[j], kk[j] * v);
          p = fmaf(S[j], qq[j], p);
        }
        p += __shfl_xor_sync(0xffffffffu, p, 4);
        p += __shfl_xor_sync(0xffffffffu, p, 8);
        p += __shfl_xor_sync(0xffffffffu, p, 16);
        o = p;
      } else {
        float g = row[2 * DIMP + SCAN_COLS], beta = row[2 * DIMP + SCAN_COLS + 1], kq = row[2 * DIMP + SCAN_COLS + 2];
        float sk = 0.f, sq = 0.f;  // S^T k and S^T q of the state before this token
#pragma unroll
        for (int j = 0; j < RPL; ++j) {
          sk = fmaf(S[j], kk[j], sk);
          sq = fmaf(S[j], qq[j], sq);
        }
        sk += __shfl_xor_sync(0xffffffffu, sk, 4);
        sq += __shfl_xor_sync(0xffffffffu, sq, 4);
        sk += __shfl_xor_sync(0xffffffffu, sk, 8);
        sq += __shfl_xor_sync(0xffffffffu, sq, 8);
        sk += __shfl_xor_sync(0xffffffffu, sk, 16);
        sq += __shfl_xor_sync(0xffffffffu, sq, 16);
        // (g S + k u^T)^T q = g S^T q + u (k . q): the read-out of the state after the write, without a second sum
        float u = beta * (v - g * sk);
        o = fmaf(g, sq, u * kq);
#pragma unroll
        for (int j = 0; j < RPL; ++j) S[j] = fmaf(kk[j], u, g * S[j]);
      }
      if (rg == 0 && col < a.vdim)
        a.out[(size_t)(first + chunk * TOKENS + t) * (a.heads * a.vdim) + head * a.vdim + col] = o;
    }
    __syncthreads();  // the stage is filled again two rounds on
  }
#pragma unroll
  for (int j = 0; j < RPL; ++j)
    if (col < a.vdim && rg * RPL + j < a.dim) my_state[j] = S[j];
}

template <int MODE>
static int launch_scan(const ScanArgs& a, int sequences, cudaStream_t stream) {
  dim3 grid((a.vdim + SCAN_COLS - 1) / SCAN_COLS, a.heads, sequences);
  int rows_per_lane = (a.dim + 7) / 8;
#define SCAN_CASE(RPL, TOKENS)                                                                                    \
  {                                                                                                               \
    size_t bytes = 2 * (size_t)TOKENS * (2 * RPL * 8 + SCAN_COLS + 4) * sizeof(float);                            \
    return dllm_launch_pdl(scan_kernel<RPL, MODE, TOKENS>, grid, dim3(SCAN_THREADS), bytes, stream, a);           \
  }
  if (rows_per_lane <= 4) SCAN_CASE(4, 16)
  if (rows_per_lane <= 8) SCAN_CASE(8, 16)
  if (rows_per_lane <= 16) SCAN_CASE(16, 16)
  SCAN_CASE(32, 8)
#undef SCAN_CASE
}

static bool scan_sizes_ok(int heads, int qk_heads, int dim, int vdim, int stride) {
  return heads > 0 && qk_heads > 0 && heads % qk_heads == 0 && dim > 0 && dim <= 256 && dim % 4 == 0 && vdim > 0 &&
         stride > 0 && heads < 65536;
}

// Decayed outer products over the new tokens of every sequence of the step. q, k, v: pointers to the first token's
// first head inside rows of `stride` floats (float32). activation 1 applies silu to q, k and v on the way in; keys
// are then multiplied by k_scale. Head h decays by decay[h] per token.
DLLM_EXPORT int dllm_decay_scan(const float* q, const float* k, const float* v, int stride, int heads, int dim,
                                int vdim, const float* decay, int activation, float k_scale, float* state,
                                const int* cu_seqlens, const int* slots, int sequences, float* out,
                                cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (!scan_sizes_ok(heads, heads, dim, vdim, stride) || sequences >= 65536) return DLLM_UNSUPPORTED_SIZE;
  if (!q || !k || !v || !decay || !state || !cu_seqlens || !slots || !out) return DLLM_BAD_ARGUMENT;
  ScanArgs a = {};
  a.q = q; a.k = k; a.v = v; a.stride = stride; a.heads = heads; a.qk_heads = heads; a.dim = dim; a.vdim = vdim;
  a.state = state; a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.decay = decay;
  a.activation = activation; a.k_scale = k_scale;
  return launch_scan<0>(a, sequences, stream);
}

// The gated delta rule over the new tokens of every sequence. q and k are unit vectors (q scaled) per q/k head, v
// the values per head, all float32 in rows of `stride` floats; aux holds per token the heads' decays g, the heads'
// step sizes beta and the q/k heads' k.q (see `dllm_delta_prepare`).
DLLM_EXPORT int dllm_delta_scan(const float* q, const float* k, const float* v, int stride, int heads, int qk_heads,
                                int dim, int vdim, const float* aux, int aux_stride, float* state,
                                const int* cu_seqlens, const int* slots, int sequences, float* out,
                                cudaStream_t stream) {
  if (sequences <= 0) return DLLM_OK;
  if (!scan_sizes_ok(heads, qk_heads, dim, vdim, stride) || sequences >= 65536) return DLLM_UNSUPPORTED_SIZE;
  if (!q || !k || !v || !aux || !state || !cu_seqlens || !slots || !out) return DLLM_BAD_ARGUMENT;
  ScanArgs a = {};
  a.q = q; a.k = k; a.v = v; a.stride = stride; a.heads = heads; a.qk_heads = qk_heads; a.dim = dim; a.vdim = vdim;
  a.state = state; a.cu_seqlens = cu_seqlens; a.slots = slots; a.out = out; a.aux = aux; a.aux_stride = aux_stride;
  a.k_scale = 1.0f;
  return launch_scan<1>(a, sequences, stream);
}

// ---- what the delta rule needs of a token before its scan --------------------------------------------------------
// proj[t] = [q (qk_heads x dim) | k (qk_heads x dim) | v (heads x vdim) | ... | b (heads) | a (heads)] float32, the
// first `channels` = 2 qk_heads dim + heads vdim of them pass a causal convolution over time per channel
// (taps[channel][j], the last column multiplying the token itself; inputs before the step come from
// conv_state[slot][taps - 1][channels], zeros before the sequence's start) and silu; q and k are then divided by
// sqrt(sum of squares + 1e-6) per head, q also multiplied by dim^(-1/2). Written: prepared[t][channels] and
// aux[t] = [g (heads) | beta (heads) | k.q (qk_heads)] with beta = sigmoid(b), g = exp(-exp(A_log) softplus(a +
// dt_bias)). In a step of single tokens (`single` != 0) the block also moves the convolution's history on.
#define DELTA_MAX_TAPS 8

struct DeltaPrepareArgs {
  const float* proj; int stride; int b_off, a_off;
  const float* taps; int n_taps;
  const float* a_log; const float* dt_bias;
  float* conv_state;
  const int* tok_seq; const int* cu_seqlens; const int* slots;
  int heads, qk_heads, dim, vdim;
  float* prepared; float* aux;
  int single;
};

__global__ void __launch_bounds__(256) delta_prepare_kernel(DeltaPrepareArgs a) {
  extern __shared__ float values[];  // [channels]
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, seq = a.tok_seq[t], local = t - a.cu_seqlens[seq], slot = a.slots[seq];
  const int qk = a.qk_heads * a.dim, channels = 2 * qk + a.heads * a.vdim, history = a.n_taps - 1;
  const float* row = a.proj + (size_t)t * a.stride;
  float* kept = a.conv_state + (size_t)slot * history * channels;
  for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) {
    float x[DELTA_MAX_TAPS];
    for (int j = 0; j < a.n_taps; ++j) {
      int back = history - j;  // how many tokens before this one
      x[j] = back <= local ? row[ch - (ptrdiff_t)back * a.stride] : kept[(size_t)(history - (back - local)) * channels + ch];
    }
    float sum = 0.f;
    for (int j = 0; j < a.n_taps; ++j) sum = fmaf(a.taps[(size_t)ch * a.n_taps + j], x[j], sum);
    values[ch] = silu_exact(sum);
    if (a.single)  // the history moves on by this token: this thread alone reads and writes the channel
      for (int j = 0; j < history; ++j) kept[(size_t)j * channels + ch] = x[j + 1];
  }
  __syncthreads();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, warps = blockDim.x >> 5;
  for (int vec = warp; vec < 2 * a.qk_heads; vec += warps) {  // q heads, then k heads
    float* p = values + vec * a.dim;
    float ss = 0.f;
    for (int i = lane; i < a.dim; i += 32) ss = fmaf(p[i], p[i], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss + 1e-6f);
    if (vec < a.qk_heads) inv *= 1.0f / sqrtf((float)a.dim);
    for (int i = lane; i < a.dim; i += 32) p[i] *= inv;
  }
  __syncthreads();
  float* prepared = a.prepared + (size_t)t * channels;
  for (int ch = threadIdx.x; ch < channels; ch += blockDim.x) prepared[ch] = values[ch];
  float* aux = a.aux + (size_t)t * (2 * a.heads + a.qk_heads);
  for (int j = warp; j < a.qk_heads; j += warps) {
    float dot = 0.f;
    for (int i = lane; i < a.dim; i += 32) dot = fmaf(values[j * a.dim + i], values[qk + j * a.dim + i], dot);
    dot = warp_sum(dot);
    if (lane == 0) aux[2 * a.heads + j] = dot;
  }
  for (int h = threadIdx.x; h < a.heads; h += blockDim.x) {
    float z = row[a.a_off + h] + a.dt_bias[h];
    float softplus = z > 20.f ? z : log1pf(expf(z));
    aux[h] = expf(-expf(a.a_log[h]) * softplus);
    aux[a.heads + h] = sigmoid_exact(row[a.b_off + h]);
  }
}

// The convolution's history after a step of any lengths: the last taps - 1 inputs of each sequence, from the step's
// rows where it has that many and from the old history before them. A thread owns a channel: it reads all it
// needs before it writes.
__global__ void __launch_bounds__(256) delta_history_kernel(DeltaPrepareArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int seq = blockIdx.x, first = a.cu_seqlens[seq], count = a.cu_seqlens[seq + 1] - first, slot = a.slots[seq];
  const int channels = 2 * a.qk_heads * a.dim + a.heads * a.vdim, history = a.n_taps - 1;
  float* kept = a.conv_state + (size_t)slot * history * channels;
  for (int ch = blockIdx.y * blockDim.x + threadIdx.x; ch < channels; ch += gridDim.y * blockDim.x) {
    float x[DELTA_MAX_TAPS];
    for (int r = 0; r < history; ++r) {
      int at = count - history + r;  // index among the step's tokens of this sequence
      x[r] = at >= 0 ? a.proj[(size_t)(first + at) * a.stride + ch] : kept[(size_t)(r + count) * channels + ch];
    }
    for (int r = 0; r < history; ++r) kept[(size_t)r * channels + ch] = x[r];
  }
}

DLLM_EXPORT int dllm_delta_prepare(const float* proj, int stride, int b_off, int a_off, const float* taps, int n_taps,
                                   const float* a_log, const float* dt_bias, float* conv_state, const int* tok_seq,
                                   const int* cu_seqlens, const int* slots, int tokens, int sequences, int heads,
                                   int qk_heads, int dim, int vdim, float* prepared, float* aux, int single,
                                   cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (n_taps < 1 || n_taps > DELTA_MAX_TAPS || !scan_sizes_ok(heads, qk_heads, dim, vdim, stride))
    return DLLM_UNSUPPORTED_SIZE;
  size_t channels = 2 * (size_t)qk_heads * dim + (size_t)heads * vdim;
  if (channels * sizeof(float) > 200 * 1024) return DLLM_UNSUPPORTED_SIZE;
  if (!proj || !taps || !a_log || !dt_bias || !tok_seq || !cu_seqlens || !slots || !prepared || !aux ||
      (n_taps > 1 && !conv_state))
    return DLLM_BAD_ARGUMENT;
  DeltaPrepareArgs a = {proj, stride, b_off, a_off, taps, n_taps, a_log, dt_bias, conv_state, tok_seq, cu_seqlens,
                        slots, heads, qk_heads, dim, vdim, prepared, aux, single};
  if (channels * sizeof(float) > 48 * 1024 &&
      cudaFuncSetAttribute(delta_prepare_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                           (int)(channels * sizeof(float))) != cudaSuccess)
    return DLLM_LAUNCH_FAILED;
  int status = dllm_launch_pdl(delta_prepare_kernel, dim3(tokens), dim3(256), channels * sizeof(float), stream, a);
  if (status != DLLM_OK || single || n_taps == 1) return status;
  int across = (int)((channels + 255) / 256);
  return dllm_launch_pdl(delta_history_kernel, dim3(sequences, across), dim3(256), 0, stream, a);
}

// ---- read-out: norm, weight and gate ----------------------------------------------------------------------------
// x [tokens, width] float32 is normed in groups of `group` values (a head's vdim, or the whole width): divided by
// sqrt(mean square + eps), times weight[i % group] if a weight is given, times gate(z) with z the token's gate
// pre-activations (rows of `gate_stride` floats; gate 1: silu, 2: sigmoid), rounded once to the output type.
template <typename T>
__global__ void __launch_bounds__(128) gated_norm_kernel(T* __restrict__ out, const float* __restrict__ x,
                                                         const float* __restrict__ weight,
                                                         const float* __restrict__ gate, int gate_stride, int width,
                                                         int group, float eps, int gate_kind) {
  __shared__ float scratch[4];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x, warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float* row = x + (size_t)t * width;
  const float* z = gate + (size_t)t * gate_stride;
  T* dst = out + (size_t)t * width;
  auto finish = [&](int i, float inv) {
    float value = row[i] * inv;
    if (weight != nullptr) value *= weight[i % group];
    value *= gate_kind == 1 ? silu_exact(z[i]) : sigmoid_exact(z[i]);
    dst[i] = from_float<T>(value);
  };
  if (group == width) {
    float ss = 0.f;
    for (int i = threadIdx.x; i < width; i += blockDim.x) ss = fmaf(row[i], row[i], ss);
    ss = warp_sum(ss);
    if (lane == 0) scratch[warp] = ss;
    __syncthreads();
    float total = scratch[0] + scratch[1] + scratch[2] + scratch[3];
    float inv = 1.0f / sqrtf(total / (float)width + eps);
    for (int i = threadIdx.x; i < width; i += blockDim.x) finish(i, inv);
    return;
  }
  for (int g = warp; g < width / group; g += 4) {
    float ss = 0.f;
    for (int i = lane; i < group; i += 32) ss = fmaf(row[g * group + i], row[g * group + i], ss);
    ss = warp_sum(ss);
    float inv = 1.0f / sqrtf(ss / (float)group + eps);
    for (int i = lane; i < group; i += 32) finish(g * group + i, inv);
  }
}

DLLM_EXPORT int dllm_gated_norm(void* out, const float* x, const float* weight, const float* gate, int gate_stride,
                                int tokens, int width, int group, float eps, int gate_kind, int out_dtype,
                                cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (width <= 0 || group <= 0 || width % group || (gate_kind != 1 && gate_kind != 2)) return DLLM_UNSUPPORTED_SIZE;
  if (!out || !x || !gate) return DLLM_BAD_ARGUMENT;
  if (out_dtype == DLLM_F32)
    return dllm_launch_pdl(gated_norm_kernel<float>, dim3(tokens), dim3(128), 0, stream, (float*)out, x, weight, gate,
                           gate_stride, width, group, eps, gate_kind);
  if (out_dtype == DLLM_BF16)
    return dllm_launch_pdl(gated_norm_kernel<__nv_bfloat16>, dim3(tokens), dim3(128), 0, stream, (__nv_bfloat16*)out,
                           x, weight, gate, gate_stride, width, group, eps, gate_kind);
  return DLLM_BAD_ARGUMENT;
}
