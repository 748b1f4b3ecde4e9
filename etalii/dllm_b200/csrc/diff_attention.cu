// Differential attention over the paged cache: every query head has TWO score maps (a query and a key of `dim` values
// each, laid out [map 1 | map 2] per head) over the same values of `vdim` values; the two softmax-weighted sums are
// combined as a1 - lambda a2, divided by their root mean square over the head, scaled, and gated per head.
//
//   map_prepare:     per token, from the float32 rows the projection left: RMS norm of every (head, map) vector of q
//                    and k with a weight shared by all of them, rotation of the first `rotary_dim` places in halves
//                    (i with i + rotary_dim / 2), q to a float32 buffer, k and v into the token's place in the cache.
//   diff_attention:  one warp per (token, query head) walks the keys the token may see (its chunk, its window, or all
//                    before it) in tiles of 32: one key a lane for both maps' scores, score <- cap tanh(score / cap),
//                    two running maxima and sums, one value place a lane for both weighted sums; all in float32. It
//                    serves whole prompts and single tokens alike; a result depends only on the token's own query and
//                    the keys it sees, not on the cut of the steps or the batch.
//   diff_attention_split: the same for steps of few tokens: the warps of a block share one (token, head) pair, each
//                    walks every WARPS-th tile, and the block combines their partial results in warp order.
//
// A cache entry holds keys of 2 * dim and values of vdim per position and kv head:
// [page][ keys: kv_head, row, 2 dim | values: kv_head, row, vdim ].
#include "common.cuh"
#include "wide_kv.cuh"

namespace {
constexpr int WARPS = 4;
constexpr int SPLIT_WARPS = 16;
constexpr int MAX_DIM = 256;     // of one map's query or key
constexpr int MAX_VDIM = 256;

template <typename T> struct Vec;
template <> struct Vec<float> { static constexpr int N = 4; };
template <> struct Vec<__nv_bfloat16> { static constexpr int N = 8; };

__device__ __forceinline__ float dot_piece(const float* q, const float* k) {
  float4 v = *(const float4*)k;
  return fmaf(q[3], v.w, fmaf(q[2], v.z, fmaf(q[1], v.y, q[0] * v.x)));
}
__device__ __forceinline__ float dot_piece(const float* q, const __nv_bfloat16* k) {
  uint4 raw = *(const uint4*)k;
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    s = fmaf(q[2 * i], x.x, s);
    s = fmaf(q[2 * i + 1], x.y, s);
  }
  return s;
}

__device__ __forceinline__ float4 load_piece(const float* k) { return *(const float4*)k; }
__device__ __forceinline__ uint4 load_piece(const __nv_bfloat16* k) { return *(const uint4*)k; }
__device__ __forceinline__ float dot_loaded(const float* q, float4 v) {
  return fmaf(q[3], v.w, fmaf(q[2], v.z, fmaf(q[1], v.y, q[0] * v.x)));
}
__device__ __forceinline__ float dot_loaded(const float* q, uint4 raw) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float s = 0.f;
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 x = __bfloat1622float2(p[i]);
    s = fmaf(q[2 * i], x.x, s);
    s = fmaf(q[2 * i + 1], x.y, s);
  }
  return s;
}

// q (shared memory, float32) . k (cache row); 16-byte pieces where the size allows (four of them asked for before the
// first is used: a lane's row is its own, so nothing else hides the loads' latency), one value at a time otherwise.
template <typename T>
__device__ __forceinline__ float dot_row(const float* q, const T* k, int n, bool pieces) {
  constexpr int N = Vec<T>::N;
  float s = 0.f;
  if (pieces) {
    int d = 0;
    for (; d + 4 * N <= n; d += 4 * N) {
      auto v0 = load_piece(k + d), v1 = load_piece(k + d + N), v2 = load_piece(k + d + 2 * N),
           v3 = load_piece(k + d + 3 * N);
      s += dot_loaded(q + d, v0);
      s += dot_loaded(q + d + N, v1);
      s += dot_loaded(q + d + 2 * N, v2);
      s += dot_loaded(q + d + 3 * N, v3);
    }
    for (; d < n; d += N) s += dot_piece(q + d, k + d);
  } else {
    for (int d = 0; d < n; ++d) s = fmaf(q[d], to_float(k[d]), s);
  }
  return s;
}

// ---- norm, rotation, cache write ------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(WARPS * 32) map_prepare_kernel(
    const float* __restrict__ rows, int ld, int q_at, int k_at, int v_at, float* __restrict__ q_out, WideKv cache,
    const float* __restrict__ q_weight, const float* __restrict__ k_weight, float eps,
    const float2* __restrict__ table, int rotary_dim, int heads, int dim, const int* __restrict__ tok_seq,
    const int* __restrict__ tok_pos, const int* __restrict__ slots, int write_cache) {
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int t = blockIdx.x;
  int unit = blockIdx.y * WARPS + warp;
  int q_units = heads * 2, k_units = cache.kv_heads * 2;
  int units = q_units + (write_cache ? k_units + cache.kv_heads : 0);
  if (unit >= units) return;
  int pos = tok_pos[t];
  const float* row = rows + (size_t)t * ld;
  if (unit >= q_units + k_units) {  // a value head: copied as it is
    int g = unit - q_units - k_units;
    int slot = slots[tok_seq[t]];
    int page = cache.page_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
    T* dst = (T*)cache.base + value_at(cache, page, g, pos % cache.page_size);
    const float* src = row + v_at + (size_t)g * cache.value_dim;
    for (int i = lane; i < cache.value_dim; i += 32) dst[i] = from_float<T>(src[i]);
    return;
  }
  bool is_q = unit < q_units;
  const float* src = row + (is_q ? q_at + (size_t)unit * dim : k_at + (size_t)(unit - q_units) * dim);
  const float* weight = is_q ? q_weight : k_weight;
  float ssq = 0.f;
  for (int i = lane; i < dim; i += 32) ssq = fmaf(src[i], src[i], ssq);
  float inv = 1.0f / sqrtf(warp_sum(ssq) / (float)dim + eps);
  int half = rotary_dim / 2;
  float* q_dst = nullptr;
  T* k_dst = nullptr;
  if (is_q) {
    q_dst = q_out + ((size_t)t * q_units + unit) * dim;
  } else {
    int ku = unit - q_units;
    int slot = slots[tok_seq[t]];
    int page = cache.page_table[(size_t)slot * cache.max_pages + pos / cache.page_size];
    k_dst = (T*)cache.base + key_at(cache, page, ku / 2, pos % cache.page_size) + (size_t)(ku & 1) * dim;
  }
  for (int i = lane; i < dim; i += 32) {
    float v = src[i] * inv * weight[i];
    if (i < rotary_dim && table != nullptr) {
      int j = i < half ? i : i - half;
      float2 cs = table[(size_t)pos * half + j];
      float a = src[j] * inv * weight[j], b = src[j + half] * inv * weight[j + half];
      v = i < half ? fmaf(a, cs.x, -(b * cs.y)) : fmaf(a, cs.y, b * cs.x);
    }
    if (is_q) q_dst[i] = v;
    else k_dst[i] = from_float<T>(v);
  }
}

// ---- the two maps over one tile of 32 keys, then the values -----------------------------------------------------------
struct MapState {
  float m[2], l[2];
  float acc[2][MAX_VDIM / 32];
};

__device__ __forceinline__ void map_init(MapState& s) {
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    s.m[m] = -INFINITY;
    s.l[m] = 0.f;
#pragma unroll
    for (int i = 0; i < MAX_VDIM / 32; ++i) s.acc[m][i] = 0.f;
  }
}

template <typename T>
__device__ __forceinline__ void map_tile(MapState& st, const float* q_s, const WideKv& cache, const int* pages, int g,
                                         int dim, int j0, int end, float scale, float softcap, bool pieces, int lane) {
  const T* base = (const T*)cache.base;
  int ps = cache.page_size, vdim = cache.value_dim;
  int j = j0 + lane;
  bool valid = j < end;
  int page = valid ? pages[j / ps] : 0;
  float s[2] = {-INFINITY, -INFINITY};
  if (valid) {
    const T* krow = base + key_at(cache, page, g, j % ps);
#pragma unroll
    for (int m = 0; m < 2; ++m) {
      float v = dot_row(q_s + m * dim, krow + m * dim, dim, pieces) * scale;
      s[m] = softcap > 0.f ? softcap * tanhf(v / softcap) : v;
    }
  }
  float p[2];
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    float m_new = fmaxf(st.m[m], warp_max(s[m]));
    p[m] = valid ? expf(s[m] - m_new) : 0.f;
    float corr = expf(st.m[m] - m_new);  // 0 on the first tile (-inf)
    st.l[m] = st.l[m] * corr + warp_sum(p[m]);
#pragma unroll
    for (int i = 0; i < MAX_VDIM / 32; ++i) st.acc[m][i] *= corr;
    st.m[m] = m_new;
  }
  int count = min(32, end - j0);
  auto one_value_row = [&](int jj) {
    float p0 = __shfl_sync(0xffffffffu, p[0], jj), p1 = __shfl_sync(0xffffffffu, p[1], jj);
    int pg = __shfl_sync(0xffffffffu, page, jj);
    const T* vrow = base + value_at(cache, pg, g, (j0 + jj) % ps);
#pragma unroll
    for (int i = 0; i < MAX_VDIM / 32; ++i) {
      int d = lane + 32 * i;
      if (d < vdim) {
        float v = to_float(vrow[d]);
        st.acc[0][i] = fmaf(p0, v, st.acc[0][i]);
        st.acc[1][i] = fmaf(p1, v, st.acc[1][i]);
      }
    }
  };
  if (count == 32) {  // a whole tile: eight rows' loads on their way at a time
#pragma unroll 8
    for (int jj = 0; jj < 32; ++jj) one_value_row(jj);
  } else {
    for (int jj = 0; jj < count; ++jj) one_value_row(jj);
  }
}

// a1 - lambda a2, over its root mean square, times out_scale and the head's gate
template <typename O>
__device__ __forceinline__ void map_finish(const MapState& st, O* orow, int vdim, float lambda, float eps,
                                           float out_scale, float gate, int lane) {
  float inv0 = 1.0f / st.l[0], inv1 = 1.0f / st.l[1];
  float o[MAX_VDIM / 32];
  float ssq = 0.f;
#pragma unroll
  for (int i = 0; i < MAX_VDIM / 32; ++i) {
    int d = lane + 32 * i;
    o[i] = d < vdim ? st.acc[0][i] * inv0 - lambda * (st.acc[1][i] * inv1) : 0.f;
    ssq = fmaf(o[i], o[i], ssq);
  }
  float factor = out_scale * gate / sqrtf(warp_sum(ssq) / (float)vdim + eps);
#pragma unroll
  for (int i = 0; i < MAX_VDIM / 32; ++i) {
    int d = lane + 32 * i;
    if (d < vdim) orow[d] = from_float<O>(o[i] * factor);
  }
}

struct DiffArgs {
  const float* q;         // [tokens, heads, 2, dim] float32, normed and rotated
  const float* gates;     // gate pre-activations: gates[t * gate_ld + head]
  int gate_ld;
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
  int tokens, heads, dim;
  float scale, softcap, lambda, eps, out_scale;
  int chunk, window;
};

template <typename T, typename O>
__global__ void __launch_bounds__(WARPS * 32) diff_attention_kernel(O* __restrict__ out, WideKv cache, DiffArgs a) {
  __shared__ __align__(16) float q_s[WARPS][2 * MAX_DIM];
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  long long item = (long long)blockIdx.x * WARPS + warp;
  if (item >= (long long)a.tokens * a.heads) return;
  int t = (int)(item / a.heads), h = (int)(item % a.heads);
  int g = h / (a.heads / cache.kv_heads);
  int pos = a.tok_pos[t];
  const int* pages = cache.page_table + (size_t)a.slots[a.tok_seq[t]] * cache.max_pages;
  const float* qrow = a.q + ((size_t)t * a.heads + h) * 2 * a.dim;
  for (int d = lane; d < 2 * a.dim; d += 32) q_s[warp][d] = qrow[d];
  __syncwarp();
  bool pieces = a.dim % Vec<T>::N == 0;
  MapState st;
  map_init(st);
  int end = pos + 1;
  for (int j0 = first_visible(pos, a.chunk, a.window); j0 < end; j0 += 32)
    map_tile<T>(st, q_s[warp], cache, pages, g, a.dim, j0, end, a.scale, a.softcap, pieces, lane);
  float z = a.gates != nullptr ? a.gates[(size_t)t * a.gate_ld + h] : INFINITY;
  float gate = 1.0f / (1.0f + expf(-z));
  map_finish(st, out + ((size_t)t * a.heads + h) * cache.value_dim, cache.value_dim, a.lambda, a.eps, a.out_scale, gate,
             lane);
}

// A block per (token, head): warp w walks tiles w, w + SPLIT_WARPS, ...; partial results meet in shared memory and
// warp 0 combines them in warp order.
template <typename T, typename O>
__global__ void __launch_bounds__(SPLIT_WARPS * 32) diff_attention_split_kernel(O* __restrict__ out, WideKv cache,
                                                                               DiffArgs a) {
  __shared__ __align__(16) float q_s[2 * MAX_DIM];
  __shared__ float part_ml[SPLIT_WARPS][4];
  extern __shared__ float part_acc[];  // [SPLIT_WARPS][2][vdim]
  pdl_launch_dependents();
  pdl_wait();
  int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  int t = blockIdx.x / a.heads, h = blockIdx.x % a.heads;
  int g = h / (a.heads / cache.kv_heads);
  int vdim = cache.value_dim;
  int pos = a.tok_pos[t];
  const int* pages = cache.page_table + (size_t)a.slots[a.tok_seq[t]] * cache.max_pages;
  const float* qrow = a.q + ((size_t)t * a.heads + h) * 2 * a.dim;
  for (int d = threadIdx.x; d < 2 * a.dim; d += blockDim.x) q_s[d] = qrow[d];
  __syncthreads();
  bool pieces = a.dim % Vec<T>::N == 0;
  MapState st;
  map_init(st);
  int end = pos + 1;
  for (int j0 = first_visible(pos, a.chunk, a.window) + 32 * warp; j0 < end; j0 += 32 * SPLIT_WARPS)
    map_tile<T>(st, q_s, cache, pages, g, a.dim, j0, end, a.scale, a.softcap, pieces, lane);
  if (lane == 0) {
    part_ml[warp][0] = st.m[0]; part_ml[warp][1] = st.l[0];
    part_ml[warp][2] = st.m[1]; part_ml[warp][3] = st.l[1];
  }
#pragma unroll
  for (int i = 0; i < MAX_VDIM / 32; ++i) {
    int d = lane + 32 * i;
    if (d < vdim) {
      part_acc[((size_t)warp * 2 + 0) * vdim + d] = st.acc[0][i];
      part_acc[((size_t)warp * 2 + 1) * vdim + d] = st.acc[1][i];
    }
  }
  __syncthreads();
  if (warp != 0) return;
  MapState total;
  map_init(total);
#pragma unroll
  for (int m = 0; m < 2; ++m) {
    float best = -INFINITY;
    for (int w = 0; w < SPLIT_WARPS; ++w) best = fmaxf(best, part_ml[w][2 * m]);
    total.m[m] = best;
    for (int w = 0; w < SPLIT_WARPS; ++w) {
      float pm = part_ml[w][2 * m];
      if (pm == -INFINITY) continue;  // (a warp without a tile)
      float f = expf(pm - best);
      total.l[m] = fmaf(part_ml[w][2 * m + 1], f, total.l[m]);
#pragma unroll
      for (int i = 0; i < MAX_VDIM / 32; ++i) {
        int d = lane + 32 * i;
        if (d < vdim) total.acc[m][i] = fmaf(part_acc[((size_t)w * 2 + m) * vdim + d], f, total.acc[m][i]);
      }
    }
  }
  float z = a.gates != nullptr ? a.gates[(size_t)t * a.gate_ld + h] : INFINITY;
  float gate = 1.0f / (1.0f + expf(-z));
  map_finish(total, out + ((size_t)t * a.heads + h) * vdim, vdim, a.lambda, a.eps, a.out_scale, gate, lane);
}

bool sizes_ok(int heads, int kv_heads, int dim, int vdim, int page_size) {
  return heads > 0 && kv_heads > 0 && heads % kv_heads == 0 && dim > 0 && dim <= MAX_DIM && vdim > 0 &&
         vdim <= MAX_VDIM && page_size > 0;
}
}  // namespace

DLLM_EXPORT int dllm_map_prepare(const float* rows, int ld, int q_at, int k_at, int v_at, float* q_out, void* cache_base,
                                 const int* page_table, int max_pages, int page_size, int heads, int kv_heads, int dim,
                                 int vdim, const float* q_weight, const float* k_weight, float eps, const float* table,
                                 int rotary_dim, const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                 int write_cache, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (!sizes_ok(heads, kv_heads, dim, vdim, page_size) || rotary_dim < 0 || rotary_dim > dim || (rotary_dim & 1))
    return DLLM_UNSUPPORTED_SIZE;
  if (rows == nullptr || q_out == nullptr || q_weight == nullptr || (write_cache && k_weight == nullptr))
    return DLLM_BAD_ARGUMENT;
  WideKv cache{cache_base, page_table, max_pages, page_size, kv_heads, 2 * dim, vdim};
  int units = heads * 2 + (write_cache ? kv_heads * 3 : 0);
  dim3 grid(tokens, (units + WARPS - 1) / WARPS);
  const float2* tab = rotary_dim > 0 ? (const float2*)table : nullptr;
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(map_prepare_kernel<float>, grid, dim3(WARPS * 32), 0, stream, rows, ld, q_at, k_at, v_at,
                           q_out, cache, q_weight, k_weight, eps, tab, rotary_dim, heads, dim, tok_seq, tok_pos, slots,
                           write_cache);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(map_prepare_kernel<__nv_bfloat16>, grid, dim3(WARPS * 32), 0, stream, rows, ld, q_at, k_at,
                           v_at, q_out, cache, q_weight, k_weight, eps, tab, rotary_dim, heads, dim, tok_seq, tok_pos,
                           slots, write_cache);
  return DLLM_BAD_ARGUMENT;
}

// `split` != 0: a block of sixteen warps per (token, head) instead of a warp.
DLLM_EXPORT int dllm_diff_attention(void* out, const float* q, const float* gates, int gate_ld, void* cache_base,
                                    const int* page_table, int max_pages, int page_size, int heads, int kv_heads, int dim,
                                    int vdim, const int* tok_seq, const int* tok_pos, const int* slots, int tokens,
                                    float scale, float softcap, float lambda, float eps, float out_scale, int chunk,
                                    int window, int split, int dtype, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  if (!sizes_ok(heads, kv_heads, dim, vdim, page_size) || chunk < 0 || window < 0) return DLLM_UNSUPPORTED_SIZE;
  if (out == nullptr || q == nullptr) return DLLM_BAD_ARGUMENT;
  WideKv cache{cache_base, page_table, max_pages, page_size, kv_heads, 2 * dim, vdim};
  DiffArgs a{q, gates, gate_ld, tok_seq, tok_pos, slots, tokens, heads, dim, scale, softcap, lambda, eps, out_scale,
             chunk, window};
  long long items = (long long)tokens * heads;
  if (split) {
    size_t smem = (size_t)SPLIT_WARPS * 2 * vdim * sizeof(float);
    dim3 grid((unsigned)items), block(SPLIT_WARPS * 32);
    if (dtype == DLLM_F32)
      return dllm_launch_pdl(diff_attention_split_kernel<float, float>, grid, block, smem, stream, (float*)out, cache, a);
    if (dtype == DLLM_BF16)
      return dllm_launch_pdl(diff_attention_split_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, smem, stream,
                             (__nv_bfloat16*)out, cache, a);
    return DLLM_BAD_ARGUMENT;
  }
  dim3 grid((unsigned)((items + WARPS - 1) / WARPS)), block(WARPS * 32);
  if (dtype == DLLM_F32)
    return dllm_launch_pdl(diff_attention_kernel<float, float>, grid, block, 0, stream, (float*)out, cache, a);
  if (dtype == DLLM_BF16)
    return dllm_launch_pdl(diff_attention_kernel<__nv_bfloat16, __nv_bfloat16>, grid, block, 0, stream,
                           (__nv_bfloat16*)out, cache, a);
  return DLLM_BAD_ARGUMENT;
}
