// Differential attention of steps of single tokens (bfloat16 cache). A block serves one token and one kv head, that is
// ALL query heads of the group and both of their score maps (an "item" is a (head, map) pair), over one stretch of the
// keys the token sees; `splits` blocks share a token's keys, and the block that finishes last combines their partial
// results in stretch order (a ticket counter: nobody waits). Keys and values come page by page (64 positions) into two
// shared-memory stages by cp.async (the next page on its way while one is worked on; two blocks share a
// multiprocessor), so a page's latency is paid once:
//
//   scores:   on the tensor cores (mma.sync m16n8k16) where dim and vdim are multiples of 16: the group's heads are the
//             rows of a tile, a warp per map and sixteen keys; else a thread per (head, key) from shared memory; then
//             scale, cap * tanh(score / cap), masks, in float32
//   softmax:  a warp per item: the page's maximum, the running maximum and sum, the weights in place of the scores
//   values:   on the tensor cores too (the items are the rows, a warp per 16 value places, the weights rounded to
//             bfloat16 as that product's operand only); else a thread per value place and part of the page
//
// and at the end a1 - weight * a2 per head, over its root mean square, times the scale and the head's gate. All of
// it float32 except the cache. A token's result does not depend on its batch mates; the stretches are cut by page
// count, so it depends on `splits` only by rounding.
#include "common.cuh"
#include "wide_kv.cuh"

namespace {
typedef __nv_bfloat16 bf16;
constexpr int THREADS = 256, WARPS = 8, PAGE = 64, MAX_ITEMS = 16, STAGES = 2;

__device__ __forceinline__ void cp_async_16(void* smem, const void* gmem) {
  unsigned s = (unsigned)__cvta_generic_to_shared(smem);
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
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

constexpr int LDP = PAGE + 8;  // a row of weights as a tensor-core operand

struct DecodeArgs {
  const float* q;      // [tokens, heads, 2, dim] float32, normed and rotated
  const float* gates;  // gates[t * gate_ld + head], or null
  int gate_ld;
  const int* tok_seq;
  const int* tok_pos;
  const int* slots;
  int heads, dim;
  float scale, softcap, lambda, eps, out_scale;
  int chunk, window, splits;
  float* partial;      // [tokens, kv_heads, splits, items, vdim + 2]
  int* tickets;        // [tokens, kv_heads], zero before and after
};

__device__ __forceinline__ float dot8(const float* q, uint4 raw) {
  const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&raw);
  float4 a = *reinterpret_cast<const float4*>(q), b = *reinterpret_cast<const float4*>(q + 4);
  float2 x0 = __bfloat1622float2(p[0]), x1 = __bfloat1622float2(p[1]), x2 = __bfloat1622float2(p[2]),
         x3 = __bfloat1622float2(p[3]);
  float s = a.x * x0.x;
  s = fmaf(a.y, x0.y, s); s = fmaf(a.z, x1.x, s); s = fmaf(a.w, x1.y, s);
  s = fmaf(b.x, x2.x, s); s = fmaf(b.y, x2.y, s); s = fmaf(b.z, x3.x, s); s = fmaf(b.w, x3.y, s);
  return s;
}

template <int ITEMS>  // items rounded up to 2, 4, 8 or 16
__global__ void __launch_bounds__(THREADS) diff_decode_kernel(bf16* __restrict__ out, WideKv cache, DecodeArgs a) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  int dim = a.dim, vdim = cache.value_dim, key_dim = cache.key_dim;
  int group = a.heads / cache.kv_heads, items = group * 2;
  int ldk = key_dim + 8;
  float* q_s = reinterpret_cast<float*>(smem_raw);                 // [group][2 dim]
  float* s_s = q_s + group * 2 * dim;                               // [items][PAGE] scores, then weights
  float* state_s = s_s + ITEMS * PAGE;                              // m[ITEMS], l[ITEMS], corr[ITEMS], (unused)
  float* red_s = state_s + 4 * ITEMS;                               // [WARPS][MAX_ITEMS / 2] sums of squares (the state
                                                                    // takes four rows: what follows starts on 16 bytes)
  bf16* k_s = reinterpret_cast<bf16*>(red_s + WARPS * (MAX_ITEMS / 2));  // [STAGES][PAGE][ldk]
  int ldv = vdim + 8, ldq = dim + 8;
  bf16* v_s = k_s + STAGES * PAGE * ldk;                            // [STAGES][PAGE][ldv]
  bf16* q_b = v_s + STAGES * PAGE * ldv;                            // [2 maps][16 rows][ldq]: the queries as an operand
  bf16* p_b = q_b + 2 * 16 * ldq;                                   // [16 rows][LDP]: a page's weights as an operand
  // With sizes that tile (16 values a step), scores and weighted sums run on the tensor cores: the group's heads are
  // the rows of the score tiles (one product per map), the items the rows of the value tiles.
  bool tensor = dim % 16 == 0 && vdim % 16 == 0;
  pdl_launch_dependents();
  pdl_wait();
  int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  int split = blockIdx.x % a.splits;
  int g = (blockIdx.x / a.splits) % cache.kv_heads;
  int t = blockIdx.x / (a.splits * cache.kv_heads);
  int pos = a.tok_pos[t];
  const int* pages = cache.page_table + (size_t)a.slots[a.tok_seq[t]] * cache.max_pages;
  int end = pos + 1, first = first_visible(pos, a.chunk, a.window);
  int page_first = first / PAGE, n_pages = (end - 1) / PAGE - page_first + 1;
  int per = (n_pages + a.splits - 1) / a.splits;
  int p_begin = page_first + split * per, p_end = min(page_first + n_pages, p_begin + per);  // this block's pages

  const float* qrow = a.q + ((size_t)t * a.heads + (size_t)g * group) * 2 * dim;
  for (int i = tid; i < group * 2 * dim; i += THREADS) q_s[i] = qrow[i];
  if (tid < ITEMS) {
    state_s[tid] = -INFINITY;
    state_s[ITEMS + tid] = 0.f;
    state_s[2 * ITEMS + tid] = 1.f;
  }
  if (tensor) {
    for (int row = warp; row < 2 * 16; row += WARPS) {  // a warp per (map, head) row
      int m = row >> 4, r = row & 15;
      for (int c = lane; c < ldq; c += 32)
        q_b[row * ldq + c] = __float2bfloat16_rn(r < group && c < dim ? qrow[(size_t)r * 2 * dim + m * dim + c] : 0.f);
    }
    for (int i = tid; i < 16 * LDP; i += THREADS) p_b[i] = __float2bfloat16_rn(0.f);
  }
  const bf16* base = (const bf16*)cache.base;
  int k_pieces = key_dim >> 3, v_pieces = vdim >> 3;
  // A page's rows are copied by warps: a row takes `k_lanes` (`v_lanes`) lanes, a power of two, so a lane finds its
  // row and piece by shifts (divisions by the piece counts cost more than the copies they would steer).
  int k_lanes = 1, v_lanes = 1;
  while (k_lanes < k_pieces && k_lanes < 32) k_lanes <<= 1;
  while (v_lanes < v_pieces && v_lanes < 32) v_lanes <<= 1;
  int k_row = tid / k_lanes, k_piece = tid % k_lanes, k_rows = THREADS / k_lanes;  // (powers of two: shifts)
  int v_row = tid / v_lanes, v_piece = tid % v_lanes, v_rows = THREADS / v_lanes;
  auto load_page = [&](int stage, int p) {
    int page = pages[p];
    const bf16* ksrc = base + key_at(cache, page, g, 0);
    const bf16* vsrc = base + value_at(cache, page, g, 0);
    for (int r = k_row; r < PAGE; r += k_rows)
      for (int c = k_piece; c < k_pieces; c += k_lanes)
        cp_async_16(k_s + (stage * PAGE + r) * ldk + c * 8, ksrc + (size_t)r * key_dim + c * 8);
    for (int r = v_row; r < PAGE; r += v_rows)
      for (int c = v_piece; c < v_pieces; c += v_lanes)
        cp_async_16(v_s + (stage * PAGE + r) * ldv + c * 8, vsrc + (size_t)r * vdim + c * 8);
  };
#pragma unroll
  for (int ahead = 0; ahead < STAGES - 1; ++ahead) {  // pages on their way before the first is used
    if (p_begin + ahead < p_end) load_page(ahead, p_begin + ahead);
    cp_async_commit();
  }

  // the value phase: parts of the page side by side where the block has more threads than value places
  int parts = 1;
  while (parts < 8 && parts * 2 * vdim <= THREADS) parts *= 2;
  int part = tid / vdim, d = tid % vdim;
  bool has_values = tid < parts * vdim;
  int j_per = PAGE / parts;
  float acc[ITEMS];
#pragma unroll
  for (int it = 0; it < ITEMS; ++it) acc[it] = 0.f;
  float tile_acc[2][2][4];  // tensor path: two groups of 16 value places a warp, rows gq and gq + 8
#pragma unroll
  for (int i = 0; i < 2; ++i)
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
      for (int r = 0; r < 4; ++r) tile_acc[i][j][r] = 0.f;
  int gq = lane >> 2, tq = lane & 3, mat = lane >> 3;
  __syncthreads();

  for (int p = p_begin; p < p_end; ++p) {
    int stage = (p - p_begin) % STAGES;
    cp_async_wait<STAGES - 2>();
    __syncthreads();  // this page has landed, and everyone is done with the stage the next load overwrites
    if (p + STAGES - 1 < p_end) load_page((stage + STAGES - 1) % STAGES, p + STAGES - 1);
    cp_async_commit();
    // scores
    if (tensor) {
      int m = warp >> 2, quarter = warp & 3;  // a warp: one map, sixteen keys
      float c[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
      for (int ks = 0; ks < dim / 16; ++ks) {
        unsigned af[4], bfr[4];
        ldmatrix_x4(af, q_b + (m * 16 + (lane & 15)) * ldq + ks * 16 + (lane >> 4) * 8);
        ldmatrix_x4(bfr, k_s + (stage * PAGE + quarter * 16 + (mat >> 1) * 8 + (lane & 7)) * ldk + m * dim + ks * 16 +
                             (mat & 1) * 8);
        mma_bf16(c[0], af, bfr[0], bfr[1]);
        mma_bf16(c[1], af, bfr[2], bfr[3]);
      }
      if (gq < group) {
#pragma unroll
        for (int nj = 0; nj < 2; ++nj)
#pragma unroll
          for (int e = 0; e < 2; ++e) {
            int key = quarter * 16 + nj * 8 + tq * 2 + e;
            int key_pos = p * PAGE + key;
            float v = c[nj][e] * a.scale;
            if (a.softcap > 0.f) v = a.softcap * tanhf(v / a.softcap);
            s_s[(gq * 2 + m) * PAGE + key] = key_pos >= first && key_pos < end ? v : -INFINITY;
          }
      }
    } else
    for (int idx = tid; idx < group * PAGE; idx += THREADS) {
      int head = idx / PAGE, key = idx % PAGE;
      int key_pos = p * PAGE + key;
      bool valid = key_pos >= first && key_pos < end;
      const bf16* krow = k_s + (stage * PAGE + key) * ldk;
      const float* qh = q_s + head * 2 * dim;
#pragma unroll
      for (int m = 0; m < 2; ++m) {
        float s = 0.f;
        for (int c = 0; c < dim; c += 8) s += dot8(qh + m * dim + c, *reinterpret_cast<const uint4*>(krow + m * dim + c));
        s *= a.scale;
        if (a.softcap > 0.f) s = a.softcap * tanhf(s / a.softcap);
        s_s[(head * 2 + m) * PAGE + key] = valid ? s : -INFINITY;
      }
    }
    __syncthreads();
    // softmax: a warp per item
    for (int it = warp; it < items; it += WARPS) {
      float s0 = s_s[it * PAGE + lane], s1 = s_s[it * PAGE + 32 + lane];
      float m_old = state_s[it];
      float m_new = fmaxf(m_old, warp_max(fmaxf(s0, s1)));
      float p0 = 0.f, p1 = 0.f, corr = 1.f;
      if (m_new != -INFINITY) {
        p0 = expf(s0 - m_new);
        p1 = expf(s1 - m_new);
        corr = expf(m_old - m_new);  // 0 on the first page with a visible key
      }
      float sum = warp_sum(p0 + p1);
      s_s[it * PAGE + lane] = p0;
      s_s[it * PAGE + 32 + lane] = p1;
      if (tensor) {
        p_b[it * LDP + lane] = __float2bfloat16_rn(p0);
        p_b[it * LDP + 32 + lane] = __float2bfloat16_rn(p1);
      }
      if (lane == 0) {
        state_s[it] = m_new;
        state_s[ITEMS + it] = state_s[ITEMS + it] * corr + sum;
        state_s[2 * ITEMS + it] = corr;
      }
    }
    __syncthreads();
    // values
    if (tensor) {
      float corr_lo = gq < items ? state_s[2 * ITEMS + gq] : 1.f, corr_hi = gq + 8 < items ? state_s[2 * ITEMS + gq + 8] : 1.f;
      unsigned af[PAGE / 16][4];
#pragma unroll
      for (int kk = 0; kk < PAGE / 16; ++kk) ldmatrix_x4(af[kk], p_b + (lane & 15) * LDP + kk * 16 + (lane >> 4) * 8);
#pragma unroll
      for (int gi = 0; gi < 2; ++gi) {
        int columns = (warp + gi * WARPS) * 16;  // this warp's gi-th group of 16 value places
        if (columns >= vdim) break;
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          tile_acc[gi][j][0] *= corr_lo; tile_acc[gi][j][1] *= corr_lo;
          tile_acc[gi][j][2] *= corr_hi; tile_acc[gi][j][3] *= corr_hi;
        }
#pragma unroll
        for (int kk = 0; kk < PAGE / 16; ++kk) {
          unsigned bfr[4];
          ldmatrix_x4_trans(bfr, v_s + (stage * PAGE + kk * 16 + (mat & 1) * 8 + (lane & 7)) * ldv + columns + (mat >> 1) * 8);
          mma_bf16(tile_acc[gi][0], af[kk], bfr[0], bfr[1]);
          mma_bf16(tile_acc[gi][1], af[kk], bfr[2], bfr[3]);
        }
      }
    } else if (has_values) {
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) acc[it] *= state_s[2 * ITEMS + it];
      const bf16* vb = v_s + (size_t)stage * PAGE * ldv + d;
      for (int j = part * j_per; j < (part + 1) * j_per; j += 4) {
        float v0 = __bfloat162float(vb[(size_t)j * ldv]), v1 = __bfloat162float(vb[(size_t)(j + 1) * ldv]);
        float v2 = __bfloat162float(vb[(size_t)(j + 2) * ldv]), v3 = __bfloat162float(vb[(size_t)(j + 3) * ldv]);
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) {
          if (it < items) {
            float4 w = *reinterpret_cast<const float4*>(s_s + it * PAGE + j);
            acc[it] = fmaf(w.x, v0, fmaf(w.y, v1, fmaf(w.z, v2, fmaf(w.w, v3, acc[it]))));
          }
        }
      }
    }
    __syncthreads();  // the weights' place is free for the next page's scores
  }
  cp_async_wait<0>();
  // the parts' sums meet in the threads of part 0 (through the key/value space, free now)
  float* meet = reinterpret_cast<float*>(k_s);  // [parts][ITEMS][vdim]
  if (tensor) {
    // the tiles' rows (items) and columns (value places) go to the threads that own a value place each
    __syncthreads();
#pragma unroll
    for (int gi = 0; gi < 2; ++gi) {
      int columns = (warp + gi * WARPS) * 16;
      if (columns >= vdim) break;
#pragma unroll
      for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int r = 0; r < 4; ++r) {
          int row = gq + (r >> 1) * 8, col = columns + j * 8 + tq * 2 + (r & 1);
          if (row < items) meet[(size_t)row * vdim + col] = tile_acc[gi][j][r];
        }
    }
    __syncthreads();
    if (tid < vdim)
#pragma unroll
      for (int it = 0; it < ITEMS; ++it)
        if (it < items) acc[it] = meet[(size_t)it * vdim + d];
    __syncthreads();  // (the space serves again below)
  } else if (parts > 1) {
    __syncthreads();
    if (has_values && part > 0)
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) meet[((size_t)part * ITEMS + it) * vdim + d] = acc[it];
    __syncthreads();
    if (tid < vdim)
      for (int other = 1; other < parts; ++other)
#pragma unroll
        for (int it = 0; it < ITEMS; ++it) acc[it] += meet[((size_t)other * ITEMS + it) * vdim + d];
  }
  bool owner = tid < vdim;  // holds place d of every item's sum

  if (a.splits > 1) {
    // leave this stretch's partial result; the last block to arrive combines all of them in stretch order
    size_t stride = (size_t)vdim + 2;
    float* mine = a.partial + (((size_t)t * cache.kv_heads + g) * a.splits + split) * items * stride;
    if (owner)
#pragma unroll
      for (int it = 0; it < ITEMS; ++it)
        if (it < items) mine[it * stride + d] = acc[it];
    if (tid < items) {
      mine[tid * stride + vdim] = state_s[tid];
      mine[tid * stride + vdim + 1] = state_s[ITEMS + tid];
    }
    __threadfence();
    __syncthreads();
    __shared__ int last;
    if (tid == 0) {
      int* ticket = a.tickets + (size_t)t * cache.kv_heads + g;
      int arrived = atomicAdd(ticket, 1);
      last = arrived == a.splits - 1;
      if (last) *ticket = 0;
    }
    __syncthreads();
    if (!last) return;
    __threadfence();
    const float* all = a.partial + ((size_t)t * cache.kv_heads + g) * a.splits * items * stride;
    // every (item, stretch)'s maximum and sum with one thread each, then each stretch's factor, then the sums: the
    // loads of a phase do not wait for one another
    float* m_all = meet;                       // [items][splits] (the key/value space again)
    float* l_all = m_all + MAX_ITEMS * 16;
    float* f_all = l_all + MAX_ITEMS * 16;
    if (tid < items * a.splits) {
      int it = tid / a.splits, s = tid % a.splits;
      m_all[tid] = __ldcg(all + ((size_t)s * items + it) * stride + vdim);
      l_all[tid] = __ldcg(all + ((size_t)s * items + it) * stride + vdim + 1);
    }
    __syncthreads();
    if (tid < items) {
      float best = -INFINITY, sum = 0.f;
      for (int s = 0; s < a.splits; ++s) best = fmaxf(best, m_all[tid * a.splits + s]);
      for (int s = 0; s < a.splits; ++s) {
        float m = m_all[tid * a.splits + s];
        float f = m == -INFINITY ? 0.f : expf(m - best);
        f_all[tid * a.splits + s] = f;
        sum = fmaf(l_all[tid * a.splits + s], f, sum);
      }
      state_s[tid] = best;
      state_s[ITEMS + tid] = sum;
    }
    __syncthreads();
    if (owner)
#pragma unroll
      for (int it = 0; it < ITEMS; ++it) {
        if (it < items) {
          float sum = 0.f;
#pragma unroll 4
          for (int s = 0; s < a.splits; ++s)
            sum = fmaf(__ldcg(all + ((size_t)s * items + it) * stride + d), f_all[it * a.splits + s], sum);
          acc[it] = sum;
        }
      }
  }
  // a1 - weight * a2 per head, its root mean square over the head, the scale and the gate
  float o[ITEMS / 2];
#pragma unroll
  for (int h = 0; h < ITEMS / 2; ++h) {
    o[h] = 0.f;
    if (owner && h < group)
      o[h] = acc[2 * h] / state_s[ITEMS + 2 * h] - a.lambda * (acc[2 * h + 1] / state_s[ITEMS + 2 * h + 1]);
    float ssq = warp_sum(o[h] * o[h]);
    if (lane == 0) red_s[warp * (MAX_ITEMS / 2) + h] = ssq;
  }
  __syncthreads();
  if (!owner) return;
#pragma unroll
  for (int h = 0; h < ITEMS / 2; ++h) {
    if (h >= group) break;
    float ssq = 0.f;
    for (int w = 0; w < WARPS; ++w) ssq += red_s[w * (MAX_ITEMS / 2) + h];
    int head = g * group + h;
    float z = a.gates != nullptr ? a.gates[(size_t)t * a.gate_ld + head] : INFINITY;
    float factor = a.out_scale / (1.0f + expf(-z)) / sqrtf(ssq / (float)vdim + a.eps);
    out[((size_t)t * a.heads + head) * vdim + d] = __float2bfloat16_rn(o[h] * factor);
  }
}

size_t shared_bytes(int group, int dim, int vdim, int items_padded) {
  size_t floats = (size_t)group * 2 * dim + (size_t)items_padded * PAGE + 4 * items_padded + WARPS * (MAX_ITEMS / 2);
  size_t stages = STAGES * (size_t)PAGE * (2 * dim + 8 + vdim + 8) * sizeof(bf16);
  size_t operands = ((size_t)2 * 16 * (dim + 8) + 16 * LDP) * sizeof(bf16);
  int parts = 1;
  while (parts < 8 && parts * 2 * vdim <= THREADS) parts *= 2;
  size_t meet = (size_t)parts * items_padded * vdim * sizeof(float);  // (shares the stages' space)
  return floats * sizeof(float) + (stages > meet ? stages : meet) + operands;
}

template <int ITEMS>
int launch(void* out, const WideKv& cache, const DecodeArgs& a, int tokens, size_t smem, cudaStream_t stream) {
  static size_t configured = 0;
  if (smem > configured) {
    if (cudaFuncSetAttribute(diff_decode_kernel<ITEMS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
        cudaSuccess)
      return DLLM_LAUNCH_FAILED;
    configured = smem;
  }
  dim3 grid((unsigned)((size_t)tokens * cache.kv_heads * a.splits));
  return dllm_launch_pdl(diff_decode_kernel<ITEMS>, grid, dim3(THREADS), smem, stream, (bf16*)out, cache, a);
}
}  // namespace

// Whether the kernel takes these sizes: 0, or the status it would return.
DLLM_EXPORT int dllm_diff_attention_decode_fits(int heads, int kv_heads, int dim, int vdim, int page_size) {
  if (heads <= 0 || kv_heads <= 0 || heads % kv_heads) return DLLM_BAD_ARGUMENT;
  int group = heads / kv_heads;
  if (group * 2 > MAX_ITEMS || dim <= 0 || (dim & 7) || vdim <= 0 || (vdim & 7) || vdim > THREADS || page_size != PAGE)
    return DLLM_UNSUPPORTED_SIZE;
  int padded = group * 2 <= 2 ? 2 : (group * 2 <= 4 ? 4 : (group * 2 <= 8 ? 8 : 16));
  return shared_bytes(group, dim, vdim, padded) <= 200 * 1024 ? DLLM_OK : DLLM_UNSUPPORTED_SIZE;
}

// out [tokens, heads * vdim] bfloat16, one token per sequence. partial: tokens * kv_heads * splits * (2 heads /
// kv_heads) * (vdim + 2) floats (unused with splits == 1); tickets: tokens * kv_heads zeros, left zero.
DLLM_EXPORT int dllm_diff_attention_decode(void* out, const float* q, const float* gates, int gate_ld, void* cache_base,
                                           const int* page_table, int max_pages, int page_size, int heads,
                                           int kv_heads, int dim, int vdim, const int* tok_seq, const int* tok_pos,
                                           const int* slots, int tokens, float scale, float softcap, float lambda,
                                           float eps, float out_scale, int chunk, int window, int splits,
                                           float* partial, int* tickets, cudaStream_t stream) {
  if (tokens <= 0) return DLLM_OK;
  int fits = dllm_diff_attention_decode_fits(heads, kv_heads, dim, vdim, page_size);
  if (fits != DLLM_OK) return fits;
  if (splits < 1 || splits > 16 || chunk < 0 || window < 0 || (splits > 1 && (partial == nullptr || tickets == nullptr)))
    return DLLM_BAD_ARGUMENT;
  WideKv cache{cache_base, page_table, max_pages, page_size, kv_heads, 2 * dim, vdim};
  DecodeArgs a{q, gates, gate_ld, tok_seq, tok_pos, slots, heads, dim, scale, softcap, lambda, eps, out_scale,
               chunk, window, splits, partial, tickets};
  int items = 2 * heads / kv_heads;
  int padded = items <= 2 ? 2 : (items <= 4 ? 4 : (items <= 8 ? 8 : 16));
  size_t smem = shared_bytes(heads / kv_heads, dim, vdim, padded);
  if (padded == 2) return launch<2>(out, cache, a, tokens, smem, stream);
  if (padded == 4) return launch<4>(out, cache, a, tokens, smem, stream);
  if (padded == 8) return launch<8>(out, cache, a, tokens, smem, stream);
  return launch<16>(out, cache, a, tokens, smem, stream);
}
