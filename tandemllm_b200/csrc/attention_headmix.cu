// Attention whose heads' weights are mixed after the softmax, over the paged cache, on the CUDA cores (32-bit or
// bfloat16 storage, 32-bit arithmetic throughout), with an optional sigmoid gate a head on the output:
//
//   s_g(i, j) = scale * <q_g(i), k_c(g)(j)>  over the keys j the row sees (max(0, i - window + 1) .. i; window 0: all)
//   p_g = softmax_j s_g;   p'_h(i, j) = sum_g M[h, g] p_g(i, j);   o_h(i) = gate_h(i) * sum_j p'_h(i, j) v_c(h)(j)
//
// (c(h) = h / (Hq / Hk): the KV head of query head h; M [Hq, Hq], row-major; gate_h = sigmoid of a logit a head.)
// The mix needs every head's finished softmax at a key, so a row's heads are worked on together and in two passes:
// the first finds each head's maximum and sum, the second forms p, mixes it with M / sum and applies it to the values.
//
// One block takes one row and one span of its keys. Keys are visited in tiles of 32 aligned to absolute positions, and
// the spans are cut from the tile that holds the row's first visible key, so the order of every addition depends on the
// row's position alone: not on how a prompt was cut, on the batch, or on the pages. With one span a single kernel does
// both passes; with several (long contexts, few rows) a first kernel leaves every span's maximum and sum, a second joins
// them, applies its span and leaves partial outputs, and a third adds those in span order.
#include <type_traits>

#include "common.cuh"

namespace tl {

constexpr int HM_TILE = 32;
constexpr int HM_THREADS = 256;

struct HeadMixParams {
  const void* q;              // [rows, Hq, D]
  const void* k_cache;        // [pages, Hk, page_size, D]
  const void* v_cache;
  const int* block_table;     // [requests, max_pages]
  int max_pages, page_size, num_pages;
  const int* req_of_row;
  const int* positions;
  float scale;
  int window;
  const float* mix;           // [Hq, Hq] or null (no mixing)
  const void* gate;           // the gate's logit of (row r, head h) at gate[r * ld_gate + h], or null
  long long ld_gate;
  void* out;                  // [rows, Hq, D]
  float* stats;               // [rows, spans, Hq, 2]: a span's maximum and sum
  float* partial;             // [rows, spans, Hq * D]
  int rows, Hq, Hk, D, spans, span_keys;
  int* status;
};

// Shared memory of a block: the row's queries and outputs in 32-bit, two tiles of weights, the mix, the heads' maxima
// and sums, and the tile's keys and values of `kc` KV heads at a time in the cache's own type (rows padded by 16 bytes,
// so that a warp's lanes, a key each, read their rows without meeting in a bank).
template <typename T> __host__ __device__ inline int headmix_row_pad(int D) {
  return D % (16 / (int)sizeof(T)) == 0 ? D + 16 / (int)sizeof(T) : D + 1;
}
template <typename T> __host__ __device__ inline size_t headmix_smem_bytes(int Hq, int D, int kc) {
  const size_t floats = (size_t)2 * Hq * D + (size_t)2 * Hq * HM_TILE + (size_t)Hq * Hq + 2 * (size_t)Hq;
  return ((floats * 4 + 15) / 16) * 16 + (size_t)2 * kc * HM_TILE * headmix_row_pad<T>(D) * sizeof(T);
}

__device__ __forceinline__ void hm_cp_async16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;          // 0: the 16 bytes are filled with zeros
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src),
               "r"(bytes) : "memory");
}
__device__ __forceinline__ void hm_cp_async_wait() {
  asm volatile("cp.async.commit_group;" ::: "memory");
  asm volatile("cp.async.wait_group 0;" ::: "memory");
}

// PHASE 0: both passes (one span). 1: the span's maximum and sum. 2: the joined statistics, then the span's outputs.
// `kc`: KV heads whose keys and values a block holds in shared memory at a time (all of them where they fit).
template <typename T, int PHASE>
__global__ void __launch_bounds__(HM_THREADS) headmix_attention_kernel(HeadMixParams p, int kc) {
  extern __shared__ __align__(16) float hm_smem[];
  const int Hq = p.Hq, Hk = p.Hk, D = p.D, group = Hq / Hk;
  float* qs = hm_smem;                         // [Hq, D]
  float* osm = qs + (size_t)Hq * D;            // [Hq, D]
  float* P = osm + (size_t)Hq * D;             // [Hq, 32]
  float* PM = P + Hq * HM_TILE;                // [Hq, 32]
  float* mixs = PM + Hq * HM_TILE;             // [Hq, Hq]: M[h, g] / sum_g
  float* ms = mixs + Hq * Hq;                  // [Hq]
  float* ls = ms + Hq;                         // [Hq]
  const int DP = headmix_row_pad<T>(D);
  const size_t head_bytes = ((((size_t)2 * Hq * D + (size_t)2 * Hq * HM_TILE + (size_t)Hq * Hq + 2 * (size_t)Hq) * 4 + 15) / 16) * 16;
  T* sK = reinterpret_cast<T*>(reinterpret_cast<char*>(hm_smem) + head_bytes);      // [kc, 32, DP]
  T* sV = sK + (size_t)kc * HM_TILE * DP;
  __shared__ long long rowoff[HM_TILE];
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, nwarps = HM_THREADS / 32;
  const int r = blockIdx.x, span = blockIdx.y;
  const int pos = p.positions[r];
  const int b = p.req_of_row[r];
  const int* table = p.block_table + (long long)b * p.max_pages;
  const int first = p.window > 0 ? max(0, pos - p.window + 1) : 0;
  const int tile0 = first / HM_TILE * HM_TILE;                 // where this row's spans begin
  const int lo = max(first, tile0 + span * p.span_keys);       // this block's keys: lo .. hi
  const int hi = min(pos, tile0 + (span + 1) * p.span_keys - 1);
  const T* Q = (const T*)p.q + (long long)r * Hq * D;
  // a row whose keys reach past the spans the launch was given: recorded, and the keys beyond are not read
  if (tid == 0 && span == 0 && pos - tile0 >= p.spans * p.span_keys) atomicExch(p.status, 6);
  for (int i = tid; i < Hq * D; i += HM_THREADS) {
    qs[i] = to_f32(Q[i]);
    if (PHASE != 1) osm[i] = 0.f;
  }
  for (int g = tid; g < Hq; g += HM_THREADS) {
    ms[g] = -INFINITY;
    ls[g] = 0.f;
  }
  __syncthreads();
  constexpr int VEC = 16 / (int)sizeof(T);
  const bool vec_ok = D % VEC == 0;
  const long long head_stride = (long long)p.page_size * D;

  // where the tile's keys lie (KV head 0; -1: not visible from this block, or no page)
  auto locate = [&](int j0) {
    if (tid < HM_TILE) {
      const int j = j0 + tid;
      long long off = -1;
      if (j >= lo && j <= hi) {
        const int page = table_page(table, j / p.page_size, p.max_pages, p.num_pages);
        if (page < 0) atomicExch(p.status, 3);
        else off = ((long long)page * Hk * p.page_size + j % p.page_size) * D;
      }
      rowoff[tid] = off;
    }
  };
  // the tile's rows of KV heads c0 .. c0 + nc - 1 from `cache` into `dst` (rows that are not seen become zeros); a thread
  // takes the same 16-byte piece of the same key for every KV head, so a piece's place is worked out once
  auto stage = [&](const T* cache, T* dst, int c0, int nc) {
    if (vec_ok) {
      const int per_row = D / VEC;
      for (int i = tid; i < HM_TILE * per_row; i += HM_THREADS) {
        const int jj = i / per_row, ch = i - jj * per_row;
        const long long off = rowoff[jj];
        const T* src = cache + (off < 0 ? 0 : off + (long long)c0 * head_stride + ch * VEC);
        T* to = dst + (size_t)jj * DP + ch * VEC;
        for (int cc = 0; cc < nc; ++cc) {
          hm_cp_async16(to, src, off >= 0);
          to += (size_t)HM_TILE * DP;
          if (off >= 0) src += head_stride;
        }
      }
    } else {
      const int n = nc * HM_TILE * D;
      for (int i = tid; i < n; i += HM_THREADS) {
        const int d = i % D, jj = (i / D) % HM_TILE, cc = i / (D * HM_TILE);
        const long long off = rowoff[jj];
        dst[((size_t)cc * HM_TILE + jj) * DP + d] = off < 0 ? from_f32<T>(0.f) : cache[off + (long long)(c0 + cc) * head_stride + d];
      }
    }
  };
  // Scores of the heads of KV heads c0 .. c0 + nc - 1 against the staged keys, a key a lane; `use(g, s)` is called by the
  // whole warp with head g's score of the lane's key (-inf where the key is not seen). HB heads of a group share each
  // piece of the key's row (HB divides the group, so the loops over them unroll without guards).
  auto scores_of = [&](auto hb_tag, int c0, int nc, auto&& use) {
    constexpr int HB = decltype(hb_tag)::value;
    const int blocks = group / HB;
    const bool seen = rowoff[lane] >= 0;
    for (int u = warp; u < nc * blocks; u += nwarps) {
      const int cc = u / blocks, g0 = (c0 + cc) * group + (u - cc * blocks) * HB;
      const T* krow = sK + ((size_t)cc * HM_TILE + lane) * DP;
      const float* q0 = qs + (size_t)g0 * D;
      float acc[HB];
#pragma unroll
      for (int i = 0; i < HB; ++i) acc[i] = 0.f;
      if (vec_ok) {
        for (int d = 0; d < D; d += VEC) {
          const uint4 raw = *reinterpret_cast<const uint4*>(krow + d);
          const T* e = reinterpret_cast<const T*>(&raw);
          float f[VEC];
#pragma unroll
          for (int x = 0; x < VEC; ++x) f[x] = to_f32(e[x]);
#pragma unroll
          for (int i = 0; i < HB; ++i) {
            const float* qg = q0 + (size_t)i * D + d;
#pragma unroll
            for (int x = 0; x < VEC; x += 4) {
              const float4 q4 = *reinterpret_cast<const float4*>(qg + x);
              acc[i] = fmaf(q4.x, f[x], acc[i]); acc[i] = fmaf(q4.y, f[x + 1], acc[i]);
              acc[i] = fmaf(q4.z, f[x + 2], acc[i]); acc[i] = fmaf(q4.w, f[x + 3], acc[i]);
            }
          }
        }
      } else {
        for (int d = 0; d < D; ++d) {
          const float f = to_f32(krow[d]);
#pragma unroll
          for (int i = 0; i < HB; ++i) acc[i] = fmaf(q0[(size_t)i * D + d], f, acc[i]);
        }
      }
#pragma unroll
      for (int i = 0; i < HB; ++i) use(g0 + i, seen ? acc[i] * p.scale : -INFINITY);
    }
  };
  // as many heads together as keep every warp busy, a power of two that divides the group
  int hb = 1;
  while (hb < 8 && group % (2 * hb) == 0 && 2 * hb <= (Hq + nwarps - 1) / nwarps) hb *= 2;
  auto scores = [&](int c0, int nc, auto&& use) {
    if (hb == 8) scores_of(std::integral_constant<int, 8>{}, c0, nc, use);
    else if (hb == 4) scores_of(std::integral_constant<int, 4>{}, c0, nc, use);
    else if (hb == 2) scores_of(std::integral_constant<int, 2>{}, c0, nc, use);
    else scores_of(std::integral_constant<int, 1>{}, c0, nc, use);
  };
  const bool whole = kc >= Hk;        // every KV head's tile fits at once: keys and values are staged together

  if (PHASE != 2) {
    for (int j0 = lo / HM_TILE * HM_TILE; j0 <= hi; j0 += HM_TILE) {
      locate(j0);
      __syncthreads();
      for (int c0 = 0; c0 < Hk; c0 += kc) {
        const int nc = min(kc, Hk - c0);
        stage((const T*)p.k_cache, sK, c0, nc);
        hm_cp_async_wait();
        __syncthreads();
        scores(c0, nc, [&](int g, float s) {
          const float tmax = warp_max(s);
          if (tmax == -INFINITY) return;
          const float m_old = ms[g], m_new = fmaxf(m_old, tmax);
          const float sum = warp_sum(s == -INFINITY ? 0.f : expf(s - m_new));
          __syncwarp();
          if (lane == 0) {
            ls[g] = (m_old == -INFINITY ? 0.f : ls[g] * expf(m_old - m_new)) + sum;
            ms[g] = m_new;
          }
          __syncwarp();
        });
        __syncthreads();
      }
    }
  }
  if (PHASE == 1) {
    float* st = p.stats + ((long long)r * p.spans + span) * Hq * 2;
    for (int g = tid; g < Hq; g += HM_THREADS) {
      st[2 * g] = ms[g];
      st[2 * g + 1] = ls[g];
    }
    return;
  }
  if (PHASE == 2) {
    // every span's maximum and sum, joined in span order
    const float* st = p.stats + (long long)r * p.spans * Hq * 2;
    for (int g = tid; g < Hq; g += HM_THREADS) {
      float m = -INFINITY;
      for (int s = 0; s < p.spans; ++s) m = fmaxf(m, st[((long long)s * Hq + g) * 2]);
      float l = 0.f;
      for (int s = 0; s < p.spans; ++s) {
        const float m_s = st[((long long)s * Hq + g) * 2], l_s = st[((long long)s * Hq + g) * 2 + 1];
        if (m_s != -INFINITY) l += l_s * expf(m_s - m);
      }
      ms[g] = m;
      ls[g] = l;
    }
    __syncthreads();
  }
  for (int i = tid; i < Hq * Hq; i += HM_THREADS) {
    const int h = i / Hq, g = i - h * Hq;
    const float w = p.mix ? p.mix[i] : (h == g ? 1.f : 0.f);
    mixs[i] = ls[g] > 0.f ? w / ls[g] : 0.f;
  }
  __syncthreads();
  for (int j0 = lo / HM_TILE * HM_TILE; j0 <= hi; j0 += HM_TILE) {
    locate(j0);
    __syncthreads();
    for (int c0 = 0; c0 < Hk; c0 += kc) {
      const int nc = min(kc, Hk - c0);
      stage((const T*)p.k_cache, sK, c0, nc);
      if (whole) stage((const T*)p.v_cache, sV, 0, Hk);
      hm_cp_async_wait();
      __syncthreads();
      scores(c0, nc, [&](int g, float s) { P[g * HM_TILE + lane] = s == -INFINITY ? 0.f : expf(s - ms[g]); });
      __syncthreads();
    }
    for (int i = tid; i < Hq * HM_TILE; i += HM_THREADS) {
      const int h = i / HM_TILE, jj = i - h * HM_TILE;
      const float* mh = mixs + h * Hq;
      float acc = 0.f;
      for (int g = 0; g < Hq; ++g) acc = fmaf(mh[g], P[g * HM_TILE + jj], acc);
      PM[i] = acc;
    }
    __syncthreads();
    const int jj_lo = max(lo - j0, 0), jj_hi = min(hi - j0, HM_TILE - 1);
    for (int c0 = 0; c0 < Hk; c0 += kc) {
      const int nc = min(kc, Hk - c0);
      if (!whole) {
        stage((const T*)p.v_cache, sV, c0, nc);
        hm_cp_async_wait();
        __syncthreads();
      }
      const int h_first = c0 * group, n_heads = nc * group;
      if (vec_ok) {
        for (int o4 = tid; o4 < n_heads * D / 4; o4 += HM_THREADS) {
          const int o = h_first * D + o4 * 4, h = o / D, d = o - h * D;
          const T* vcol = sV + ((size_t)(h / group - c0) * HM_TILE) * DP + d;
          const float* w = PM + h * HM_TILE;
          float4 acc = *reinterpret_cast<const float4*>(osm + o);
#pragma unroll 4
          for (int jj = jj_lo; jj <= jj_hi; ++jj) {
            const T* v = vcol + (size_t)jj * DP;
            if constexpr (sizeof(T) == 4) {
              const float4 x = *reinterpret_cast<const float4*>(v);
              acc.x = fmaf(w[jj], x.x, acc.x); acc.y = fmaf(w[jj], x.y, acc.y);
              acc.z = fmaf(w[jj], x.z, acc.z); acc.w = fmaf(w[jj], x.w, acc.w);
            } else {
              const uint2 raw = *reinterpret_cast<const uint2*>(v);
              const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
              const float2 a = __bfloat1622float2(h2[0]), c2 = __bfloat1622float2(h2[1]);
              acc.x = fmaf(w[jj], a.x, acc.x); acc.y = fmaf(w[jj], a.y, acc.y);
              acc.z = fmaf(w[jj], c2.x, acc.z); acc.w = fmaf(w[jj], c2.y, acc.w);
            }
          }
          *reinterpret_cast<float4*>(osm + o) = acc;
        }
      } else {
        for (int oi = tid; oi < n_heads * D; oi += HM_THREADS) {
          const int o = h_first * D + oi, h = o / D, d = o - h * D;
          const T* vcol = sV + ((size_t)(h / group - c0) * HM_TILE) * DP + d;
          float acc = osm[o];
          for (int jj = jj_lo; jj <= jj_hi; ++jj) acc = fmaf(PM[h * HM_TILE + jj], to_f32(vcol[(size_t)jj * DP]), acc);
          osm[o] = acc;
        }
      }
      __syncthreads();
    }
  }
  if (PHASE == 2) {
    float* dst = p.partial + ((long long)r * p.spans + span) * Hq * D;
    for (int o = tid; o < Hq * D; o += HM_THREADS) dst[o] = osm[o];
    return;
  }
  T* out = (T*)p.out + (long long)r * Hq * D;
  const T* gate = p.gate ? (const T*)p.gate + (long long)r * p.ld_gate : nullptr;
  for (int o = tid; o < Hq * D; o += HM_THREADS) {
    const float g = gate ? 1.f / (1.f + expf(-to_f32(gate[o / D]))) : 1.f;
    out[o] = from_f32<T>(osm[o] * g);
  }
}

// out = gate * (the spans' partial outputs added in span order)
template <typename T>
__global__ void __launch_bounds__(256) headmix_join_kernel(HeadMixParams p) {
  // a thread an output element: its spans' partial results are independent loads, all in flight together
  const int r = blockIdx.x, n = p.Hq * p.D;
  const int o = blockIdx.y * blockDim.x + threadIdx.x;
  if (o >= n) return;
  const float* src = p.partial + (long long)r * p.spans * n + o;
  float acc = 0.f;
  int s = 0;
  for (; s + 8 <= p.spans; s += 8) {
    float v[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) v[i] = src[(long long)(s + i) * n];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc += v[i];
  }
  for (; s < p.spans; ++s) acc += src[(long long)s * n];
  const T* gate = p.gate ? (const T*)p.gate + (long long)r * p.ld_gate : nullptr;
  const float g = gate ? 1.f / (1.f + expf(-to_f32(gate[o / p.D]))) : 1.f;
  ((T*)p.out)[(long long)r * n + o] = from_f32<T>(acc * g);
}

template <typename T>
static int headmix_launch(const HeadMixParams& p, cudaStream_t stream) {
  // as many KV heads' tiles at a time as keep a block within 110 KB (two blocks an SM), one at least
  int kc = p.Hk;
  while (kc > 1 && headmix_smem_bytes<T>(p.Hq, p.D, kc) > 110 * 1024) kc = (kc + 1) / 2;
  const size_t smem = headmix_smem_bytes<T>(p.Hq, p.D, kc);
  TL_REQUIRE(smem <= 200 * 1024, "head-mixed attention: %d heads of size %d need %zu bytes of shared memory a block",
             p.Hq, p.D, smem);
  dim3 grid(p.rows, p.spans);
#define TL_HM(PHASE_)                                                                                                  \
  do {                                                                                                                 \
    if (smem > 48 * 1024) {                                                                                            \
      cudaError_t e_ = cudaFuncSetAttribute(headmix_attention_kernel<T, PHASE_>,                                       \
                                            cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                   \
      if (e_ != cudaSuccess) return (int)e_;                                                                           \
    }                                                                                                                  \
    headmix_attention_kernel<T, PHASE_><<<grid, HM_THREADS, smem, stream>>>(p, kc);                                      \
    TL_LAUNCH_CHECK();                                                                                                 \
  } while (0)
  if (p.spans == 1) {
    TL_HM(0);
    return 0;
  }
  TL_HM(1);
  TL_HM(2);
#undef TL_HM
  headmix_join_kernel<T><<<dim3(p.rows, ceil_div(p.Hq * p.D, 256)), 256, 0, stream>>>(p);
  TL_LAUNCH_CHECK();
  return 0;
}

}  // namespace tl

using namespace tl;

// Spans of `span_keys` keys that cover what a row can see: `window` keys (0: all) up to a context of `max_context`, from
// the 32-key tile that holds its first one.
extern "C" int tl_headmix_spans(int max_context, int window, int span_keys) {
  int reach = max_context;
  if (window > 0 && window + HM_TILE - 1 < reach) reach = window + HM_TILE - 1;
  return reach <= 0 || span_keys <= 0 ? 1 : ceil_div(reach, span_keys);
}

// Floats of scratch for `spans` > 1: the statistics, then the partial outputs.
extern "C" long long tl_headmix_scratch_floats(int rows, int Hq, int D, int spans) {
  return spans <= 1 ? 0 : (long long)rows * spans * Hq * (2 + D);
}

extern "C" int tl_attention_headmix(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                    int max_pages, int page_size, int num_pages, const int* req_of_row,
                                    const int* positions, float scale, int window, const float* mix, const void* gate,
                                    long long ld_gate, void* out, float* scratch, int rows, int Hq, int Hk, int D, int spans,
                                    int span_keys, int dtype, int* status, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(Hq > 0 && Hk > 0 && Hq % Hk == 0, "head-mixed attention: %d query heads over %d KV heads", Hq, Hk);
  TL_REQUIRE(D > 0 && D <= 1024, "head-mixed attention: head size %d", D);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "head-mixed attention: page size %d, table width %d, window %d",
             page_size, max_pages, window);
  TL_REQUIRE(spans >= 1 && spans <= 65535 && span_keys > 0 && span_keys % HM_TILE == 0,
             "head-mixed attention: %d spans of %d keys (multiples of %d)", spans, span_keys, HM_TILE);
  TL_REQUIRE(spans == 1 || scratch, "head-mixed attention: %d spans and no scratch", spans);
  HeadMixParams p;
  p.q = q; p.k_cache = k_cache; p.v_cache = v_cache; p.block_table = block_table; p.max_pages = max_pages;
  p.page_size = page_size; p.num_pages = num_pages; p.req_of_row = req_of_row; p.positions = positions; p.scale = scale;
  p.window = window; p.mix = mix; p.gate = gate; p.ld_gate = ld_gate; p.out = out;
  p.stats = scratch; p.partial = scratch ? scratch + (long long)rows * spans * Hq * 2 : nullptr;
  p.rows = rows; p.Hq = Hq; p.Hk = Hk; p.D = D; p.spans = spans; p.span_keys = span_keys; p.status = status;
  return dtype == TL_FP32 ? headmix_launch<float>(p, stream) : headmix_launch<bf16>(p, stream);
}
