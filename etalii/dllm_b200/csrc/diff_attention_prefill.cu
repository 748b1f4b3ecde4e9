// Differential attention of prompt-sized steps on the tensor cores (bfloat16, mma.sync m16n8k16), blockwise with an
// online softmax per map. A block takes 64 consecutive new tokens of one sequence and one query head. Its eight warps
// form two groups of four, one per score map: a group holds its map's queries, walks every key tile the tile's
// tokens may see (whole cache pages of 64 positions, its map's half of the key rows and the values, cp.async, double
// buffered), and keeps its map's running maximum, sum and weighted sum of values. At the end the second group's sum
// goes through shared memory to the first, which forms a1 - weight * a2, divides by the root mean square over the
// head, applies the scale and the head's gate and stores. Scores (float32 accumulators of bfloat16 products), the cap
// cap * tanh(score / cap), the softmax and the combination are float32; weights are rounded to bfloat16 only as the
// operand of the second product. Masks: causal, chunks counted from position 0, and a window, per element.
//
// dim and vdim: multiples of 8 up to 128 (instantiated for 32, 64, 128 and padded with zeros). Pages of 64.
#include "common.cuh"
#include "wide_kv.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int BM = 64, BN = 64, WARPS = 4, MAPS = 2, THREADS = MAPS * WARPS * 32;
constexpr int MAX_TILES = 512;  // page indices kept in shared memory; beyond: read as needed
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem, bool valid) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }
__device__ __forceinline__ void ldmatrix_x4(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldmatrix_x4_trans(unsigned* r, const void* p) {
  unsigned s = (unsigned)__cvta_generic_to_shared(p);
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_bf16(float* c, const unsigned* a, unsigned b0, unsigned b1) {
  asm volatile(
      "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
      : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
      : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// 1 / x with the hardware approximation (about one unit in the last place; 1 / inf = 0).
__device__ __forceinline__ float fast_rcp(float x) {
  float y;
  asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<unsigned*>(&v);
}

struct PrefillArgs {
  const float* q;      // [tokens, heads, 2, dim] float32, normed and rotated
  const float* gates;  // gates[t * gate_ld + head], or null
  int gate_ld;
  const int* tile_seq;
  const int* tile_first;
  const int* cu_seqlens;
  const int* start;
  const int* slots;
  int heads, dim;
  float scale, softcap, lambda, eps, out_scale;
  int chunk, window;
};

template <int DQ, int DV>
__global__ void __launch_bounds__(THREADS) diff_prefill_kernel(bf16* __restrict__ out, WideKv cache, PrefillArgs a) {
  constexpr int LDQ = DQ + 8, LDV = DV + 8;  // padded rows, 16-byte aligned
  extern __shared__ __align__(16) unsigned char smem_raw[];
  bf16* q_all = reinterpret_cast<bf16*>(smem_raw);                           // [MAPS][BM][LDQ]
  int map = threadIdx.x / (WARPS * 32);
  bf16* q_s = q_all + (size_t)map * BM * LDQ;
  bf16* k_s = q_all + MAPS * BM * LDQ + (size_t)map * (2 * BN * LDQ + 2 * BN * LDV);  // [2][BN][LDQ]
  bf16* v_s = k_s + 2 * BN * LDQ;                                             // [2][BN][LDV]
  int tile = blockIdx.x, h = blockIdx.y;
  int b = a.tile_seq[tile], q0 = a.tile_first[tile];
  int dim = a.dim, vdim = cache.value_dim, heads = a.heads;
  int g = h / (heads / cache.kv_heads);
  int n_new = a.cu_seqlens[b + 1] - a.cu_seqlens[b];
  int tok0 = a.cu_seqlens[b] + q0;
  int rows = min(BM, n_new - q0);
  int pos0 = a.start[b] + q0;
  const int* pages = cache.page_table + (size_t)a.slots[b] * cache.max_pages;
  const bf16* base = (const bf16*)cache.base;
  int tid = threadIdx.x % (WARPS * 32), lane = tid & 31, warp = tid >> 5;  // within the group
  int q_pieces = dim >> 3, v_pieces = vdim >> 3;                           // 16-byte pieces of a real row
  auto group_sync = [&]() { asm volatile("bar.sync %0, %1;" ::"r"(map + 1), "r"(WARPS * 32) : "memory"); };

  // queries of both maps -> shared memory as bfloat16 (rows beyond the tile and places beyond dim are zero)
  for (int idx = threadIdx.x; idx < MAPS * BM * (DQ / 8); idx += THREADS) {
    int m = idx / (BM * (DQ / 8)), rest = idx % (BM * (DQ / 8));
    int r = rest / (DQ / 8), c = rest % (DQ / 8);
    uint4 packed = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows && c < q_pieces) {
      const float* src = a.q + (((size_t)(tok0 + r) * heads + h) * 2 + m) * dim + c * 8;
      float4 lo = *reinterpret_cast<const float4*>(src), hi = *reinterpret_cast<const float4*>(src + 4);
      packed = make_uint4(pack_bf16(lo.x, lo.y), pack_bf16(lo.z, lo.w), pack_bf16(hi.x, hi.y), pack_bf16(hi.z, hi.w));
    }
    *reinterpret_cast<uint4*>(q_all + ((size_t)m * BM + r) * LDQ + c * 8) = packed;
  }
  int last_pos = pos0 + rows - 1;
  int kt_end = last_pos / BN;
  int kt_begin = first_visible(pos0, a.chunk, a.window) / BN;
  __shared__ int page_s[MAX_TILES];
  for (int i = threadIdx.x; i <= kt_end - kt_begin && i < MAX_TILES; i += THREADS) page_s[i] = pages[kt_begin + i];
  __syncthreads();

  auto load_kv = [&](int stage, int kt) {
    int page = kt - kt_begin < MAX_TILES ? page_s[kt - kt_begin] : pages[kt];
    const bf16* ksrc = base + key_at(cache, page, g, 0) + (size_t)map * dim;  // this map's half of the key rows
    const bf16* vsrc = base + value_at(cache, page, g, 0);
    for (int idx = tid; idx < BN * (DQ / 8); idx += WARPS * 32) {
      int r = idx / (DQ / 8), c = idx % (DQ / 8);
      bool ok = c < q_pieces;
      cp_async_16(k_s + (stage * BN + r) * LDQ + c * 8, ok ? ksrc + (size_t)r * cache.key_dim + c * 8 : ksrc, ok);
    }
    for (int idx = tid; idx < BN * (DV / 8); idx += WARPS * 32) {
      int r = idx / (DV / 8), c = idx % (DV / 8);
      bool ok = c < v_pieces;
      cp_async_16(v_s + (stage * BN + r) * LDV + c * 8, ok ? vsrc + (size_t)r * vdim + c * 8 : vsrc, ok);
    }
  };
  load_kv(0, kt_begin);
  cp_async_commit();

  float o_acc[DV / 8][4];
#pragma unroll
  for (int i = 0; i < DV / 8; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) o_acc[i][j] = 0.f;
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  unsigned q_frag[DQ / 16][4];
#pragma unroll
  for (int ks = 0; ks < DQ / 16; ++ks)
    ldmatrix_x4(q_frag[ks], q_s + (warp * 16 + (lane & 15)) * LDQ + ks * 16 + (lane >> 4) * 8);
  int gq = lane >> 2, tq = lane & 3;
  int row_pos[2] = {pos0 + warp * 16 + gq, pos0 + warp * 16 + gq + 8};
  int row_first[2] = {first_visible(row_pos[0], a.chunk, a.window), first_visible(row_pos[1], a.chunk, a.window)};
  int warp_last_first = first_visible(pos0 + warp * 16 + 15, a.chunk, a.window);  // the warp's latest first key
  // Scores are kept in units of log2 e (the softmax then needs no multiplication before its exponential). With a cap:
  // cap tanh(x / cap) = cap - 2 cap / (e^(2 x / cap) + 1), so score' = cap_at - cap_twice / (2^(s * in_scale) + 1).
  bool capped = a.softcap > 0.f;
  float in_scale = capped ? a.scale * 2.0f * LOG2E / a.softcap : a.scale * LOG2E;
  float cap_at = a.softcap * LOG2E, cap_twice = -2.0f * a.softcap * LOG2E;

  for (int kt = kt_begin; kt <= kt_end; ++kt) {
    int stage = (kt - kt_begin) & 1;
    if (kt + 1 <= kt_end) load_kv(stage ^ 1, kt + 1);
    cp_async_commit();
    cp_async_wait<1>();
    group_sync();
    float s[BN / 8][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) s[j][r] = 0.f;
    const bf16* kb = k_s + stage * BN * LDQ;
#pragma unroll
    for (int ks = 0; ks < DQ / 16; ++ks) {
#pragma unroll
      for (int jp = 0; jp < BN / 16; ++jp) {
        unsigned bfr[4];
        int mat = lane >> 3;
        ldmatrix_x4(bfr, kb + (jp * 16 + (mat >> 1) * 8 + (lane & 7)) * LDQ + ks * 16 + (mat & 1) * 8);
        mma_bf16(s[2 * jp], q_frag[ks], bfr[0], bfr[1]);
        mma_bf16(s[2 * jp + 1], q_frag[ks], bfr[2], bfr[3]);
      }
    }
    // scale, cap (in units of log2 e), masks
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) {
        float v = s[j][r] * in_scale;
        if (capped) v = fmaf(cap_twice, fast_rcp(fast_exp2(v) + 1.0f), cap_at);
        s[j][r] = v;
      }
    int key0 = kt * BN;
    bool need_mask = key0 + BN - 1 > pos0 + warp * 16 || key0 < warp_last_first;
    if (need_mask) {
#pragma unroll
      for (int j = 0; j < BN / 8; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int key = key0 + j * 8 + tq * 2 + (r & 1);
          if (key > row_pos[r >> 1] || key < row_first[r >> 1]) s[j][r] = -INFINITY;
        }
    }
    float tile_max[2] = {-INFINITY, -INFINITY};
#pragma unroll
    for (int j = 0; j < BN / 8; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) tile_max[r >> 1] = fmaxf(tile_max[r >> 1], s[j][r]);
    float corr[2];
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 1));
      tile_max[i] = fmaxf(tile_max[i], __shfl_xor_sync(0xffffffffu, tile_max[i], 2));
      float m_new = fmaxf(m_run[i], tile_max[i]);
      float m_use = m_new == -INFINITY ? 0.f : m_new;  // a row that sees nothing in this tile (and nothing before)
      corr[i] = fast_exp2(m_run[i] - m_use);
      m_run[i] = m_new;
      tile_max[i] = m_use;
    }
    float row_sum[2] = {0.f, 0.f};
    unsigned p_frag[BN / 16][4];
#pragma unroll
    for (int j = 0; j < BN / 8; ++j) {
      float p0 = fast_exp2(s[j][0] - tile_max[0]), p1 = fast_exp2(s[j][1] - tile_max[0]);
      float p2 = fast_exp2(s[j][2] - tile_max[1]), p3 = fast_exp2(s[j][3] - tile_max[1]);
      row_sum[0] += p0 + p1;
      row_sum[1] += p2 + p3;
      p_frag[j >> 1][(j & 1) * 2 + 0] = pack_bf16(p0, p1);
      p_frag[j >> 1][(j & 1) * 2 + 1] = pack_bf16(p2, p3);
    }
#pragma unroll
    for (int i = 0; i < 2; ++i) l_run[i] = l_run[i] * corr[i] + row_sum[i];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      o_acc[i][0] *= corr[0]; o_acc[i][1] *= corr[0];
      o_acc[i][2] *= corr[1]; o_acc[i][3] *= corr[1];
    }
    const bf16* vb = v_s + stage * BN * LDV;
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
#pragma unroll
      for (int np = 0; np < DV / 16; ++np) {
        unsigned bfr[4];
        int mat = lane >> 3;
        ldmatrix_x4_trans(bfr, vb + (kk * 16 + (mat & 1) * 8 + (lane & 7)) * LDV + np * 16 + (mat >> 1) * 8);
        mma_bf16(o_acc[2 * np], p_frag[kk], bfr[0], bfr[1]);
        mma_bf16(o_acc[2 * np + 1], p_frag[kk], bfr[2], bfr[3]);
      }
    }
    group_sync();  // the stage is free for the load after next
  }
  cp_async_wait<0>();
#pragma unroll
  for (int i = 0; i < 2; ++i) {
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 1);
    l_run[i] += __shfl_xor_sync(0xffffffffu, l_run[i], 2);
  }
  // the second map's sums go to the first map's group through shared memory (the key/value space is free now)
  __syncthreads();
  float* ex_o = reinterpret_cast<float*>(q_all + MAPS * BM * LDQ);  // [DV / 8 * 4][WARPS * 32]
  float* ex_l = ex_o + (size_t)WARPS * 32 * (DV / 2);                // [2][WARPS * 32]
  if (map == 1) {
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
#pragma unroll
      for (int j = 0; j < 4; ++j) ex_o[(size_t)(i * 4 + j) * (WARPS * 32) + tid] = o_acc[i][j];
    ex_l[tid] = l_run[0];
    ex_l[WARPS * 32 + tid] = l_run[1];
  }
  __syncthreads();
  if (map == 1) return;
#pragma unroll
  for (int half = 0; half < 2; ++half) {
    int r = warp * 16 + gq + half * 8;
    float inv_first = 1.0f / l_run[half];
    float inv_second = a.lambda / ex_l[half * WARPS * 32 + tid];
    float ssq = 0.f;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i)
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        int j = half * 2 + c;
        float o = o_acc[i][j] * inv_first - ex_o[(size_t)(i * 4 + j) * (WARPS * 32) + tid] * inv_second;
        o_acc[i][j] = o;
        ssq = fmaf(o, o, ssq);
      }
    ssq += __shfl_xor_sync(0xffffffffu, ssq, 1);
    ssq += __shfl_xor_sync(0xffffffffu, ssq, 2);
    if (r >= rows) continue;
    float z = a.gates != nullptr ? a.gates[(size_t)(tok0 + r) * a.gate_ld + h] : INFINITY;
    float factor = a.out_scale / (1.0f + expf(-z)) / sqrtf(ssq / (float)vdim + a.eps);
    bf16* dst = out + ((size_t)(tok0 + r) * heads + h) * vdim;
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) {
      int d = i * 8 + tq * 2;
      if (d < vdim) *reinterpret_cast<__nv_bfloat162*>(dst + d) =
          __floats2bfloat162_rn(o_acc[i][half * 2] * factor, o_acc[i][half * 2 + 1] * factor);
    }
  }
}

template <int DQ, int DV>
int launch(void* out, const WideKv& cache, const PrefillArgs& a, int tiles, cudaStream_t stream) {
  size_t smem = (size_t)(MAPS * BM * (DQ + 8) + MAPS * (2 * BN * (DQ + 8) + 2 * BN * (DV + 8))) * sizeof(bf16);
  static bool configured = false;
  if (!configured) {
    if (cudaFuncSetAttribute(diff_prefill_kernel<DQ, DV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = true;
  }
  dim3 grid(tiles, a.heads);
  diff_prefill_kernel<DQ, DV><<<grid, THREADS, smem, stream>>>((bf16*)out, cache, a);
  return dllm_launch_status();
}

template <int DQ>
int launch_values(void* out, const WideKv& cache, const PrefillArgs& a, int tiles, cudaStream_t stream) {
  if (cache.value_dim <= 32) return launch<DQ, 32>(out, cache, a, tiles, stream);
  if (cache.value_dim <= 64) return launch<DQ, 64>(out, cache, a, tiles, stream);
  return launch<DQ, 128>(out, cache, a, tiles, stream);
}
}  // namespace

// out [tokens, heads * vdim] bfloat16; q [tokens, heads * 2 * dim] float32. tile_seq / tile_first: for each tile of up
// to 64 new tokens, its sequence and the index of its first token among the sequence's new tokens. The keys and
// values of the new tokens are already in the cache.
DLLM_EXPORT int dllm_diff_attention_prefill(void* out, const float* q, const float* gates, int gate_ld,
                                            void* cache_base, const int* page_table, int max_pages, int page_size,
                                            int heads, int kv_heads, int dim, int vdim, const int* tile_seq,
                                            const int* tile_first, const int* cu_seqlens, const int* start,
                                            const int* slots, int tiles, float scale, float softcap, float lambda,
                                            float eps, float out_scale, int chunk, int window, cudaStream_t stream) {
  if (tiles <= 0) return DLLM_OK;
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads || chunk < 0 || window < 0) return DLLM_BAD_ARGUMENT;
  if (dim <= 0 || dim > 128 || (dim & 7) || vdim <= 0 || vdim > 128 || (vdim & 7) || page_size != BN || heads > 65535)
    return DLLM_UNSUPPORTED_SIZE;
  WideKv cache{cache_base, page_table, max_pages, page_size, kv_heads, 2 * dim, vdim};
  PrefillArgs a{q, gates, gate_ld, tile_seq, tile_first, cu_seqlens, start, slots, heads, dim, scale, softcap, lambda,
                eps, out_scale, chunk, window};
  if (dim <= 32) return launch_values<32>(out, cache, a, tiles, stream);
  if (dim <= 64) return launch_values<64>(out, cache, a, tiles, stream);
  return launch_values<128>(out, cache, a, tiles, stream);
}
