// Head-mixed attention for prompt portions in bfloat16 on the tensor cores (mma.sync m16n8k16, 32-bit accumulation):
//
//   s_g(i, j) = scale * <q_g(i), k_c(g)(j)>,  p_g = softmax_j s_g over the keys row i sees (its window),
//   p'_h = sum_g M[h, g] p_g,   o_h(i) = sigmoid(gate_h(i)) * sum_j p'_h(i, j) v_c(h)(j)
//
// One block of NW (eight or sixteen) warps takes 16 consecutive query rows of one request and ALL heads, because the mix
// needs every head's finished softmax at a (row, key). A warp owns up to HPW heads (head = warp + NW i); sixteen warps
// where eight would hold four heads' outputs each (one block an SM either way: twice the warps to cover latencies). Keys are visited in tiles of
// 32 aligned to absolute positions, twice:
//   pass 1   S = Q K^T on the tensor cores, each head's running maximum and sum a row in registers (32-bit)
//   pass 2   S again; p = exp(s - max) / sum in 32-bit into shared memory; every thread mixes the heads of its (row, key)
//            places in 32-bit FMAs (the mix is part of the weights, which stay 32-bit until they are applied); the mixed
//            weights are rounded to bfloat16 as the A operand of O += P' V, V read as it lies in the cache
// A tile's keys (and values) of all KV heads are staged with cp.async, 16-byte chunks XOR-swizzled by the row for
// ldmatrix. The order of a row's additions depends on its position alone. Head sizes 64 and 128.
#include "common.cuh"

namespace tl {
namespace hmm {

constexpr int BM = 16;          // query rows a block
constexpr int TJ = 32;          // keys a tile
constexpr int PS = 40;          // floats a row of a head's weight tile (16 x 32 used): 64-bit accesses of a half warp
                                // (rows r .. r + 3, four column pairs each) then fall into 32 different banks

__device__ __forceinline__ uint32_t saddr(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
  const int bytes = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(saddr(dst)), "l"(src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most N of this thread's committed groups are still in flight (the most recent ones)
template <int N> __device__ __forceinline__ void cp_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }
__device__ __forceinline__ void ldsm4(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void ldsm4t(uint32_t addr, uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float* c, uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack2(float lo, float hi) {
  __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&v);
}
// byte offset of 16-byte chunk `chunk` of row `row` in a tile whose rows hold D bfloat16
template <int D> __device__ __forceinline__ int swz(int row, int chunk) { return row * (D * 2) + ((chunk ^ (row & 7)) << 4); }

struct Params {
  const bf16* q; const bf16* k_cache; const bf16* v_cache;
  const int* block_table; int max_pages, page_size, num_pages;
  const int* tiles;           // [n, 3] = (request, first row, rows <= 16)
  const int* positions;
  float scale; int window;
  const float* mix;           // [Hq, Hq] or null
  const bf16* gate; long long ld_gate;
  bf16* out;
  int Hq, Hk;
  int* status;
};

template <int D> __host__ __device__ inline size_t smem_bytes(int Hq, int Hk) {
  const size_t hq_max = (size_t)(Hq + 7) / 8 * 8 <= 8 ? 8 : ((Hq + 7) / 8 <= 2 ? 16 : 32);     // 8 x heads a warp
  return (size_t)Hq * BM * D * 2 + (size_t)2 * Hk * TJ * D * 2 + (size_t)Hq * BM * PS * 4 + hq_max * hq_max * 4;
}

template <int D, int HPW, int NW>
__global__ void __launch_bounds__(NW * 32, (NW == 16 || HPW * D >= 256) ? 1 : 2) headmix_mma_kernel(Params p) {
  constexpr int THREADS = NW * 32;
  constexpr int CH = D / 8;                    // 16-byte chunks a row
  constexpr int HQMAX = NW * HPW;
  extern __shared__ __align__(128) uint8_t hmm_smem[];
  const int Hq = p.Hq, Hk = p.Hk, group = Hq / Hk;
  uint8_t* sQ = hmm_smem;                                       // [Hq][16][D] bf16
  uint8_t* sK = sQ + (size_t)Hq * BM * D * 2;                   // [Hk][32][D]
  uint8_t* sV = sK + (size_t)Hk * TJ * D * 2;                   // [Hk][32][D]
  float* sP = reinterpret_cast<float*>(sV + (size_t)Hk * TJ * D * 2);      // [Hq][16][PS]
  float* sM = sP + (size_t)Hq * BM * PS;                        // [HQMAX][HQMAX], zeros beyond the model's heads
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int t = blockIdx.x;
  const int b = p.tiles[3 * t], row0 = p.tiles[3 * t + 1], nq = min(p.tiles[3 * t + 2], BM);
  const int pos0 = p.positions[row0];
  const int* table = p.block_table + (long long)b * p.max_pages;
  const int k_lo = p.window > 0 ? max(0, pos0 - p.window + 1) : 0;
  const int k_hi = pos0 + nq - 1;

  // ---- the tile's queries, all heads; rows past the tile's are zeros ----
  for (int i = tid; i < Hq * BM * CH; i += THREADS) {
    const int c = i % CH, m = (i / CH) % BM, g = i / (CH * BM);
    const bool valid = m < nq;
    cp16(sQ + (size_t)g * BM * D * 2 + swz<D>(m, c), p.q + ((long long)(row0 + (valid ? m : 0)) * Hq + g) * D + c * 8, valid);
  }
  for (int i = tid; i < HQMAX * HQMAX; i += THREADS) {
    const int h = i / HQMAX, g = i % HQMAX;
    sM[i] = (h < Hq && g < Hq) ? (p.mix ? p.mix[h * Hq + g] : (h == g ? 1.f : 0.f)) : 0.f;
  }

  // A thread copies the same 16-byte chunk of the same key for every KV head: the key's page is looked up once a tile.
  constexpr int STAGERS = THREADS < TJ * CH ? THREADS : TJ * CH;        // threads that copy (a block may have more than chunks)
  static_assert(STAGERS % CH == 0 && (TJ * CH) % STAGERS == 0, "whole keys a round of the copying threads");
  const long long kv_head_stride = (long long)p.page_size * D;
  auto stage = [&](const bf16* cache, uint8_t* dst, int j0) {
    if (tid >= STAGERS) return;
    const int c = tid % CH;
#pragma unroll
    for (int rnd = 0; rnd < TJ * CH / STAGERS; ++rnd) {
      const int jj = tid / CH + rnd * (STAGERS / CH);
      const int kp = j0 + jj;
      bool valid = kp >= k_lo && kp <= k_hi;
      long long off = 0;
      if (valid) {
        const int pg = kp / p.page_size;
        const int page = table_page(table, pg, p.max_pages, p.num_pages);
        if (page < 0) {
          atomicExch(p.status, 3);
          valid = false;
        } else {
          off = ((long long)page * Hk * p.page_size + (kp - pg * p.page_size)) * D + c * 8;
        }
      }
      uint8_t* to = dst + swz<D>(jj, c);
      const bf16* from = cache + off;
      for (int cc = 0; cc < Hk; ++cc) cp16(to + (size_t)cc * TJ * D * 2, valid ? from + cc * kv_head_stride : cache, valid);
    }
  };
  // S = Q_g K_c^T for the tile: s[n][0..1] row lane / 4, keys 8 n + 2 (lane % 4) + {0, 1}; s[n][2..3] row lane / 4 + 8
  auto qk = [&](int g, const uint8_t* keys, float (*s)[4]) {
    const uint8_t* q_tile = sQ + (size_t)g * BM * D * 2;
    const uint8_t* k_tile = keys + (size_t)(g / group) * TJ * D * 2;
#pragma unroll
    for (int n = 0; n < 4; ++n) s[n][0] = s[n][1] = s[n][2] = s[n][3] = 0.f;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
      uint32_t a0, a1, a2, a3;
      ldsm4(saddr(q_tile + swz<D>(lane & 15, kk * 2 + (lane >> 4))), a0, a1, a2, a3);
#pragma unroll
      for (int n = 0; n < 4; n += 2) {
        uint32_t b0, b1, b2, b3;
        const int row = (n + (lane >> 4)) * 8 + (lane & 7), c = kk * 2 + ((lane >> 3) & 1);
        ldsm4(saddr(k_tile + swz<D>(row, c)), b0, b1, b2, b3);
        mma16816(s[n], a0, a1, a2, a3, b0, b1);
        mma16816(s[n + 1], a0, a1, a2, a3, b2, b3);
      }
    }
  };
  // the rows of this lane and what they see
  const int r_lo = lane >> 2, r_hi = r_lo + 8;
  const bool v_lo = r_lo < nq, v_hi = r_hi < nq;
  const int p_lo = pos0 + r_lo, p_hi = pos0 + r_hi;
  const int w_lo = p.window > 0 ? p_lo - p.window + 1 : 0, w_hi = p.window > 0 ? p_hi - p.window + 1 : 0;
  // (most tiles of a prompt lie before every row of the block and inside every row's window: nothing to mask there)
  const int open_from = p.window > 0 ? pos0 + nq - p.window : 0;
  auto mask_scale = [&](float (*s)[4], int j0) {
    if (nq == BM && j0 >= open_from && j0 >= 0 && j0 + TJ - 1 <= pos0) {
#pragma unroll
      for (int n = 0; n < 4; ++n) {
        s[n][0] *= p.scale; s[n][1] *= p.scale; s[n][2] *= p.scale; s[n][3] *= p.scale;
      }
      return;
    }
#pragma unroll
    for (int n = 0; n < 4; ++n) {
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const int kp = j0 + n * 8 + (lane & 3) * 2 + e;
        s[n][e] = (v_lo && kp <= p_lo && kp >= w_lo && kp >= 0) ? s[n][e] * p.scale : -INFINITY;
        s[n][2 + e] = (v_hi && kp <= p_hi && kp >= w_hi && kp >= 0) ? s[n][2 + e] * p.scale : -INFINITY;
      }
    }
  };

  float m_run[HPW][2], l_run[HPW][2];
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    m_run[i][0] = m_run[i][1] = -INFINITY;
    l_run[i][0] = l_run[i][1] = 0.f;
  }
  const int j_first = k_lo / TJ * TJ;

  // ---- pass 1: every head's maximum and sum a row ----
  // (the values' tile is not needed yet: it serves as a second tile of keys, so that a tile loads while the one before
  // it is worked on)
  stage(p.k_cache, sK, j_first);
  cp_commit();
  int cur = 0;
  for (int j0 = j_first; j0 <= k_hi; j0 += TJ, cur ^= 1) {
    if (j0 + TJ <= k_hi) {
      stage(p.k_cache, cur ? sK : sV, j0 + TJ);
      cp_commit();
      cp_wait<1>();
    } else {
      cp_wait<0>();
    }
    __syncthreads();
    const uint8_t* keys = cur ? sV : sK;
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int g = warp + NW * i;
      if (g < Hq) {
        float s[4][4];
        qk(g, keys, s);
        mask_scale(s, j0);
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          mx0 = fmaxf(mx0, fmaxf(s[n][0], s[n][1]));
          mx1 = fmaxf(mx1, fmaxf(s[n][2], s[n][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float n0 = fmaxf(m_run[i][0], mx0), n1 = fmaxf(m_run[i][1], mx1);
        // a row that has seen no key yet keeps 0 as its reference, so that exp(-inf - reference) is 0 and not NaN
        const float c0 = n0 == -INFINITY ? 0.f : n0, c1 = n1 == -INFINITY ? 0.f : n1;
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          sum0 += __expf(s[n][0] - c0) + __expf(s[n][1] - c0);
          sum1 += __expf(s[n][2] - c1) + __expf(s[n][3] - c1);
        }
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 1);
        sum0 += __shfl_xor_sync(0xffffffffu, sum0, 2);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 1);
        sum1 += __shfl_xor_sync(0xffffffffu, sum1, 2);
        l_run[i][0] = l_run[i][0] * expf(m_run[i][0] - c0) + sum0;
        l_run[i][1] = l_run[i][1] * expf(m_run[i][1] - c1) + sum1;
        m_run[i][0] = n0;
        m_run[i][1] = n1;
      }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    l_run[i][0] = l_run[i][0] > 0.f ? 1.f / l_run[i][0] : 0.f;
    l_run[i][1] = l_run[i][1] > 0.f ? 1.f / l_run[i][1] : 0.f;
    if (m_run[i][0] == -INFINITY) m_run[i][0] = 0.f;
    if (m_run[i][1] == -INFINITY) m_run[i][1] = 0.f;
  }

  float o[HPW][D / 8][4];
#pragma unroll
  for (int i = 0; i < HPW; ++i)
#pragma unroll
    for (int n = 0; n < D / 8; ++n) o[i][n][0] = o[i][n][1] = o[i][n][2] = o[i][n][3] = 0.f;

  // ---- pass 2: the weights, mixed over the heads, applied to the values ----
  // The next tile's keys load while this tile's weights are mixed and applied, the next tile's values while the next
  // scores are formed: a thread's copies complete in the order of their groups, keys (j), values (j), keys (j + 1), ...
  stage(p.k_cache, sK, j_first);
  cp_commit();
  stage(p.v_cache, sV, j_first);
  cp_commit();
  for (int j0 = j_first; j0 <= k_hi; j0 += TJ) {
    const bool more = j0 + TJ <= k_hi;
    cp_wait<1>();                       // this tile's keys
    __syncthreads();
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int g = warp + NW * i;
      if (g < Hq) {
        float s[4][4];
        qk(g, sK, s);
        mask_scale(s, j0);
        float* pg = sP + (size_t)g * BM * PS;
#pragma unroll
        for (int n = 0; n < 4; ++n) {
          const int col = n * 8 + (lane & 3) * 2;
          *reinterpret_cast<float2*>(pg + r_lo * PS + col) =
              make_float2(__expf(s[n][0] - m_run[i][0]) * l_run[i][0], __expf(s[n][1] - m_run[i][0]) * l_run[i][0]);
          *reinterpret_cast<float2*>(pg + r_hi * PS + col) =
              make_float2(__expf(s[n][2] - m_run[i][1]) * l_run[i][1], __expf(s[n][3] - m_run[i][1]) * l_run[i][1]);
        }
      }
    }
    __syncthreads();
    if (more) {
      stage(p.k_cache, sK, j0 + TJ);
      cp_commit();
    }
    if (p.mix) {
      // a thread owns one or two (row, key) places and mixes all heads there: p'_h = sum_g M[h, g] p_g, in place. The
      // mix's rows are read 16 bytes at a time (the same address for every thread), each value used for every place.
      constexpr int PLACES = BM * TJ / THREADS;
      static_assert(PLACES == 1 || PLACES == 2, "one or two places a thread");
      float* at0 = sP + (tid / TJ) * PS + tid % TJ;
      float* at1 = at0 + (THREADS / TJ) * PS;
      float pa[HQMAX], pb[PLACES == 2 ? HQMAX : 1];
#pragma unroll
      for (int g = 0; g < HQMAX; ++g) {
        pa[g] = g < Hq ? at0[(size_t)g * BM * PS] : 0.f;
        if constexpr (PLACES == 2) pb[g] = g < Hq ? at1[(size_t)g * BM * PS] : 0.f;
      }
      for (int h = 0; h < Hq; ++h) {
        const float4* mh = reinterpret_cast<const float4*>(sM + h * HQMAX);
        float acc_a = 0.f, acc_b = 0.f;
#pragma unroll
        for (int g4 = 0; g4 < HQMAX / 4; ++g4) {
          const float4 m4 = mh[g4];
          acc_a = fmaf(m4.x, pa[4 * g4], acc_a); acc_a = fmaf(m4.y, pa[4 * g4 + 1], acc_a);
          acc_a = fmaf(m4.z, pa[4 * g4 + 2], acc_a); acc_a = fmaf(m4.w, pa[4 * g4 + 3], acc_a);
          if constexpr (PLACES == 2) {
            acc_b = fmaf(m4.x, pb[4 * g4], acc_b); acc_b = fmaf(m4.y, pb[4 * g4 + 1], acc_b);
            acc_b = fmaf(m4.z, pb[4 * g4 + 2], acc_b); acc_b = fmaf(m4.w, pb[4 * g4 + 3], acc_b);
          }
        }
        at0[(size_t)h * BM * PS] = acc_a;
        if constexpr (PLACES == 2) at1[(size_t)h * BM * PS] = acc_b;
      }
    }
    if (more) cp_wait<1>();             // this tile's values (the next tile's keys may still be on their way)
    else cp_wait<0>();
    __syncthreads();
#pragma unroll
    for (int i = 0; i < HPW; ++i) {
      const int h = warp + NW * i;
      if (h < Hq) {
        const float* ph = sP + (size_t)h * BM * PS;
        const uint8_t* v_tile = sV + (size_t)(h / group) * TJ * D * 2;
#pragma unroll
        for (int ks = 0; ks < TJ / 16; ++ks) {
          const int col = ks * 16 + (lane & 3) * 2;
          const float2 x0 = *reinterpret_cast<const float2*>(ph + r_lo * PS + col);
          const float2 x1 = *reinterpret_cast<const float2*>(ph + r_hi * PS + col);
          const float2 x2 = *reinterpret_cast<const float2*>(ph + r_lo * PS + col + 8);
          const float2 x3 = *reinterpret_cast<const float2*>(ph + r_hi * PS + col + 8);
          const uint32_t a0 = pack2(x0.x, x0.y), a1 = pack2(x1.x, x1.y), a2 = pack2(x2.x, x2.y), a3 = pack2(x3.x, x3.y);
#pragma unroll
          for (int np = 0; np < D / 16; ++np) {
            uint32_t b0, b1, b2, b3;
            const int row = ks * 16 + (lane & 7) + 8 * ((lane >> 3) & 1), c = np * 2 + (lane >> 4);
            ldsm4t(saddr(v_tile + swz<D>(row, c)), b0, b1, b2, b3);
            mma16816(o[i][2 * np], a0, a1, a2, a3, b0, b1);
            mma16816(o[i][2 * np + 1], a0, a1, a2, a3, b2, b3);
          }
        }
      }
    }
    __syncthreads();
    if (more) {
      stage(p.v_cache, sV, j0 + TJ);
      cp_commit();
    }
  }

  // ---- gate and store ----
#pragma unroll
  for (int i = 0; i < HPW; ++i) {
    const int h = warp + NW * i;
    if (h < Hq) {
      float g_lo = 1.f, g_hi = 1.f;
      if (p.gate) {
        if (v_lo) g_lo = 1.f / (1.f + expf(-__bfloat162float(p.gate[(long long)(row0 + r_lo) * p.ld_gate + h])));
        if (v_hi) g_hi = 1.f / (1.f + expf(-__bfloat162float(p.gate[(long long)(row0 + r_hi) * p.ld_gate + h])));
      }
#pragma unroll
      for (int n = 0; n < D / 8; ++n) {
        const int d = n * 8 + (lane & 3) * 2;
        if (v_lo)
          *reinterpret_cast<uint32_t*>(p.out + ((long long)(row0 + r_lo) * Hq + h) * D + d) = pack2(o[i][n][0] * g_lo, o[i][n][1] * g_lo);
        if (v_hi)
          *reinterpret_cast<uint32_t*>(p.out + ((long long)(row0 + r_hi) * Hq + h) * D + d) = pack2(o[i][n][2] * g_hi, o[i][n][3] * g_hi);
      }
    }
  }
}

template <int D, int HPW, int NW>
static int launch(const Params& p, int n_tiles, cudaStream_t stream) {
  const size_t smem = smem_bytes<D>(p.Hq, p.Hk);
  if (smem > 48 * 1024) {          // (asked for at every launch: the attribute belongs to the current device)
    cudaError_t e = cudaFuncSetAttribute(headmix_mma_kernel<D, HPW, NW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
  }
  headmix_mma_kernel<D, HPW, NW><<<n_tiles, NW * 32, smem, stream>>>(p);
  TL_LAUNCH_CHECK();
  return 0;
}

}  // namespace hmm
}  // namespace tl

using namespace tl;

// Whether the tensor-core kernel takes these sizes: head size 64 with up to 32 heads or 128 with up to 16, pages of a
// multiple of 16 tokens (any), and a block's tiles within the shared memory of an SM.
extern "C" int tl_attention_headmix_mma_supported(int Hq, int Hk, int D) {
  if (Hq <= 0 || Hk <= 0 || Hq % Hk) return 0;
  if (D == 64) return Hq <= 32 && hmm::smem_bytes<64>(Hq, Hk) <= 227 * 1024;
  if (D == 128) return Hq <= 16 && hmm::smem_bytes<128>(Hq, Hk) <= 227 * 1024;
  return 0;
}

extern "C" int tl_attention_headmix_mma_tile_rows() { return hmm::BM; }

extern "C" int tl_attention_headmix_mma(const void* q, const void* k_cache, const void* v_cache, const int* block_table,
                                        int max_pages, int page_size, int num_pages, const int* tiles, int n_tiles,
                                        const int* positions, float scale, int window, const float* mix, const void* gate,
                                        long long ld_gate, void* out, int Hq, int Hk, int D, int* status,
                                        cudaStream_t stream) {
  if (n_tiles == 0) return 0;
  TL_REQUIRE(tl_attention_headmix_mma_supported(Hq, Hk, D), "head-mixed attention on the tensor cores: %d heads over %d of size %d",
             Hq, Hk, D);
  TL_REQUIRE(page_size > 0 && max_pages > 0 && window >= 0, "head-mixed attention: page size %d, table width %d, window %d",
             page_size, max_pages, window);
  hmm::Params p;
  p.q = (const bf16*)q; p.k_cache = (const bf16*)k_cache; p.v_cache = (const bf16*)v_cache; p.block_table = block_table;
  p.max_pages = max_pages; p.page_size = page_size; p.num_pages = num_pages; p.tiles = tiles; p.positions = positions;
  p.scale = scale; p.window = window; p.mix = mix; p.gate = (const bf16*)gate; p.ld_gate = ld_gate; p.out = (bf16*)out;
  p.Hq = Hq; p.Hk = Hk; p.status = status;
  if (D == 64) {
    if (Hq <= 8) return hmm::launch<64, 1, 8>(p, n_tiles, stream);
    if (Hq <= 16) return hmm::launch<64, 2, 8>(p, n_tiles, stream);
    // up to 32 heads: eight warps of four heads each (sixteen warps of two heads measured the same, 5.03 against 4.97 ms
    // for twelve layers of a 2048-token prompt: this case is not short of warps)
    return hmm::launch<64, 4, 8>(p, n_tiles, stream);
  }
  if (Hq <= 8) return hmm::launch<128, 1, 8>(p, n_tiles, stream);
  // up to 16 heads of 128: sixteen warps, one head each (5.61 against 6.21 ms with eight warps of two heads)
  return hmm::launch<128, 1, 16>(p, n_tiles, stream);
}
