// A selective state-space mixer's kernels (the Mamba-2 recurrence), all 32-bit:
//
//   causal_conv_act   y[t, c] = act(bias[c] + sum_k taps[c, k] u[t - (K - 1) + k, c])   per channel, inputs before a step from
//                     the request's state slot (its last K - 1 inputs), zeros before position 0 (an admitted slot is zero)
//   conv_state        the slot's K - 1 inputs after the step
//   ssm_scan          per head h (group g = h / (H / G)), state S [N, P]:
//                       dt = softplus(dt_raw + dt_bias[h]);  S <- exp(-exp(A_log[h]) dt) S + dt B_t x_t^T;  y_t = S^T C_t + D[h] x_t
//                     token by token in position order, from the request's slot, which receives the state after the step
//   gated_group_norm  v = y * silu(z); each of `groups` equal parts of a row divided by its own root mean square; times w
//
// A step's rows are several requests' portions side by side (one row for a decoding request): every kernel takes the
// row's request from req_of_row / row_start and never looks at another request's rows. The recurrence is sequential in
// a request and parallel over requests, heads and the state's columns, with a fixed order of additions, so a position's
// result does not depend on how the sequence was cut into steps or on what else is in the batch.
#include "common.cuh"

namespace tl {

// four bytes from global to shared memory without a register in between; the caller commits and waits for the group
__device__ __forceinline__ void copy_async4(float* to_shared, const float* from_global) {
  asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"((uint32_t)__cvta_generic_to_shared(to_shared)), "l"(from_global)
               : "memory");
}

__device__ __forceinline__ float silu_f(float x) { return x / (1.f + expf(-x)); }
__device__ __forceinline__ float softplus_f(float x) { return x > 20.f ? x : log1pf(expf(x)); }

#define TL_CONV_ACT_NONE 0
#define TL_CONV_ACT_SILU 1

// grid (ceil(C / 256), rows): a thread a (row, channel)
__global__ void __launch_bounds__(256) causal_conv_act_kernel(
    const float* __restrict__ in, long long ld_in, const float* __restrict__ taps, const float* __restrict__ bias,
    const float* __restrict__ state, long long state_stride, const int* __restrict__ state_slot,
    const int* __restrict__ req_of_row, const int* __restrict__ row_start, float* __restrict__ out, long long ld_out,
    int C, int K, int act) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int r = blockIdx.y;
  if (c >= C) return;
  const int b = req_of_row[r];
  const int first = row_start[b];
  const float* st = state + (long long)state_slot[b] * state_stride;        // [K - 1, C], oldest first
  float acc = bias ? bias[c] : 0.f;
  for (int k = 0; k < K; ++k) {
    const int back = K - 1 - k;             // tap k multiplies the input `back` tokens ago
    const int src = r - back;
    float u;
    if (src >= first) u = in[(long long)src * ld_in + c];
    else u = st[(long long)(K - 1 + (src - first)) * C + c];
    acc = fmaf(taps[(long long)c * K + k], u, acc);
  }
  out[(long long)r * ld_out + c] = act == TL_CONV_ACT_SILU ? silu_f(acc) : acc;
}

// grid (ceil(C / 256), requests): a thread a (request, channel) shifts the slot's K - 1 inputs
__global__ void __launch_bounds__(256) conv_state_kernel(const float* __restrict__ in, long long ld_in, float* __restrict__ state,
                                                         long long state_stride, const int* __restrict__ state_slot,
                                                         const int* __restrict__ row_start, int C, int K) {
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  if (c >= C) return;
  const int first = row_start[b], n = row_start[b + 1] - first;
  if (n <= 0) return;
  float* st = state + (long long)state_slot[b] * state_stride;
  for (int j = 0; j < K - 1; ++j) {
    // the input (K - 1 - j) tokens before the end of the step
    const int rel = n - (K - 1) + j;        // its row, counted from the step's first row
    st[(long long)j * C + c] = rel >= 0 ? in[(long long)(first + rel) * ld_in + c] : st[(long long)(j + n) * C + c];
  }
}

struct ScanParams {
  const float* xbc;          // [rows, ld_xbc]: x [H P] | B [G N] | C [G N], after the convolution and its activation
  long long ld_xbc;
  const float* dt;           // [rows, ld_dt]: the H raw step sizes of a row begin at dt
  long long ld_dt;
  const float* dt_bias;      // [H]
  const float* a_log;        // [H]
  const float* d_skip;       // [H]
  float* state;              // a slot's recurrent state [H, P, N] begins at state + slot * state_stride
  long long state_stride;
  const int* state_slot;
  const int* row_start;
  float* y;                  // [rows, H P]
  int H, P, N, G;
  int write_state;
  // Long portions are cut into chunks of `chunk_tokens` rows that run side by side (0: a request's rows one after the other):
  //   mode 1: every chunk runs from a zero state, writes no y, and leaves its last state and the product of its decays;
  //   (tl_ssm_chunk_states then walks a request's chunks: each chunk's slot receives the state the chunk starts from,
  //   S <- decay_c S + last_c, and the request's slot the state after the last chunk)
  //   mode 2: every chunk runs from the state it starts from and writes its y.
  int mode, chunk_tokens, max_chunks;
  float* chunk_state;        // [requests * max_chunks, H, P, N]
  float* chunk_decay;        // [requests * max_chunks, H]
};

constexpr int SCAN_LANES = 8;       // lanes that share a column of the state: lane l holds n = l, l + 8, ...
constexpr int SCAN_COLS = 16;       // columns (values of p) a block
constexpr int SCAN_TOKENS = 16;     // tokens staged at a time

// grid (ceil(P / 16), H, requests), 128 threads: thread (col, lane) holds NPER entries of column p of S: with VEC (the
// state's rows a multiple of 4) entries 4 lane .. 4 lane + 3 of every run of 32, read from shared memory 16 bytes at a
// time, else entries lane, lane + 8, ...
template <int NPER, bool VEC>
__global__ void __launch_bounds__(SCAN_COLS * SCAN_LANES) ssm_scan_kernel(ScanParams p) {
  // Two buffers of 16 tokens each: while one is computed on, the next 16 tokens' B, C, x and raw step sizes are on
  // their way into the other (cp.async), so that the recurrence does not wait for global memory.
  extern __shared__ __align__(16) float sm[];
  const int N = p.N, P = p.P;
  const int buf_floats = 2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_COLS + 3 * SCAN_TOKENS;
  const int h = blockIdx.y, b = blockIdx.z;
  const int col = threadIdx.x / SCAN_LANES, lane = threadIdx.x % SCAN_LANES;
  const int pcol = blockIdx.x * SCAN_COLS + col;
  const bool live = pcol < P;
  const int g = h / (p.H / p.G);
  int first, n_rows;
  float* st;
  float* chunk_decay = nullptr;
  if (p.mode == 0) {
    first = p.row_start[b];
    n_rows = p.row_start[b + 1] - first;
    st = p.state + (long long)p.state_slot[b] * p.state_stride + ((long long)h * P + (live ? pcol : 0)) * N;
  } else {
    const int req = b / p.max_chunks, c = b - req * p.max_chunks;
    first = p.row_start[req] + c * p.chunk_tokens;
    n_rows = min(p.chunk_tokens, p.row_start[req + 1] - first);
    st = p.chunk_state + ((long long)b * p.H * P + (long long)h * P + (live ? pcol : 0)) * N;
    chunk_decay = p.chunk_decay + (long long)b * p.H + h;
  }
  if (n_rows <= 0) return;
  float S[NPER];
#pragma unroll
  for (int i = 0; i < NPER; ++i) {
    const int n = VEC ? ((i >> 2) * 32 + lane * 4 + (i & 3)) : (lane + SCAN_LANES * i);
    S[i] = (live && n < N && p.mode != 1) ? st[n] : 0.f;
  }
  float decay_product = 1.f;
  const float neg_a = -expf(p.a_log[h]), bias = p.dt_bias[h], skip = p.d_skip[h];
  const long long xoff = (long long)h * P + (long long)blockIdx.x * SCAN_COLS;
  const long long boff = (long long)p.H * P + (long long)g * N;
  const long long coff = boff + (long long)p.G * N;
  auto stage = [&](int t0, int which) {
    float* base = sm + which * buf_floats;
    float* tB = base;
    float* tC = tB + SCAN_TOKENS * N;
    float* tX = tC + SCAN_TOKENS * N;
    float* tRaw = tX + SCAN_TOKENS * SCAN_COLS;
    const int nt = min(SCAN_TOKENS, n_rows - t0);
    for (int t = 0; t < nt; ++t) {
      const float* src = p.xbc + (long long)(first + t0 + t) * p.ld_xbc;
      for (int n = threadIdx.x; n < N; n += blockDim.x) {
        copy_async4(tB + t * N + n, src + boff + n);
        if (p.mode != 1) copy_async4(tC + t * N + n, src + coff + n);
      }
    }
    for (int i = threadIdx.x; i < nt * SCAN_COLS; i += blockDim.x) {
      const int t = i / SCAN_COLS, c = i - t * SCAN_COLS;
      if (blockIdx.x * SCAN_COLS + c < P) copy_async4(tX + i, p.xbc + (long long)(first + t0 + t) * p.ld_xbc + xoff + c);
      else tX[i] = 0.f;
    }
    if ((int)threadIdx.x < nt) copy_async4(tRaw + threadIdx.x, p.dt + (long long)(first + t0 + threadIdx.x) * p.ld_dt + h);
    asm volatile("cp.async.commit_group;" ::: "memory");
  };
  stage(0, 0);
  for (int t0 = 0, which = 0; t0 < n_rows; t0 += SCAN_TOKENS, which ^= 1) {
    const int nt = min(SCAN_TOKENS, n_rows - t0);
    const bool more = t0 + SCAN_TOKENS < n_rows;
    if (more) stage(t0 + SCAN_TOKENS, which ^ 1);       // (the other buffer was last read before the sync that ended the pass before this one)
    if (more) asm volatile("cp.async.wait_group 1;" ::: "memory");
    else asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    float* sB = sm + which * buf_floats;
    float* sC = sB + SCAN_TOKENS * N;
    float* sX = sC + SCAN_TOKENS * N;
    float* sRaw = sX + SCAN_TOKENS * SCAN_COLS;
    float* sDt = sRaw + SCAN_TOKENS;
    float* sA = sDt + SCAN_TOKENS;
    if ((int)threadIdx.x < nt) {
      const float d = softplus_f(sRaw[threadIdx.x] + bias);
      sDt[threadIdx.x] = d;
      sA[threadIdx.x] = expf(neg_a * d);
    }
    __syncthreads();
    if (p.mode == 1) {              // the chunk's end state and its decays' product are all that is wanted
      for (int t = 0; t < nt; ++t) {
        const float a = sA[t];
        const float dx = sDt[t] * sX[t * SCAN_COLS + col];
        const float* Bt = sB + t * N;
        decay_product *= a;
        if constexpr (VEC) {
#pragma unroll
          for (int j = 0; j < NPER / 4; ++j) {
            const int n = j * 32 + lane * 4;
            if (n < N) {
              const float4 b4 = *reinterpret_cast<const float4*>(Bt + n);
              S[4 * j] = fmaf(a, S[4 * j], dx * b4.x);
              S[4 * j + 1] = fmaf(a, S[4 * j + 1], dx * b4.y);
              S[4 * j + 2] = fmaf(a, S[4 * j + 2], dx * b4.z);
              S[4 * j + 3] = fmaf(a, S[4 * j + 3], dx * b4.w);
            }
          }
        } else {
#pragma unroll
          for (int i = 0; i < NPER; ++i) {
            const int n = lane + SCAN_LANES * i;
            if (n < N) S[i] = fmaf(a, S[i], dx * Bt[n]);
          }
        }
      }
      __syncthreads();            // the buffer may be filled again
      continue;
    }
    for (int t = 0; t < nt; ++t) {
      const float a = sA[t], x = sX[t * SCAN_COLS + col];
      const float dx = sDt[t] * x;
      const float* Bt = sB + t * N;
      const float* Ct = sC + t * N;
      float acc = 0.f;
      if constexpr (VEC) {
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
        for (int j = 0; j < NPER / 4; ++j) {
          const int n = j * 32 + lane * 4;
          if (n < N) {
            const float4 b4 = *reinterpret_cast<const float4*>(Bt + n);
            const float4 c4 = *reinterpret_cast<const float4*>(Ct + n);
            S[4 * j] = fmaf(a, S[4 * j], dx * b4.x);
            S[4 * j + 1] = fmaf(a, S[4 * j + 1], dx * b4.y);
            S[4 * j + 2] = fmaf(a, S[4 * j + 2], dx * b4.z);
            S[4 * j + 3] = fmaf(a, S[4 * j + 3], dx * b4.w);
            a0 = fmaf(S[4 * j], c4.x, a0);
            a1 = fmaf(S[4 * j + 1], c4.y, a1);
            a2 = fmaf(S[4 * j + 2], c4.z, a2);
            a3 = fmaf(S[4 * j + 3], c4.w, a3);
          }
        }
        acc = (a0 + a1) + (a2 + a3);
      } else {
#pragma unroll
        for (int i = 0; i < NPER; ++i) {
          const int n = lane + SCAN_LANES * i;
          if (n < N) {
            S[i] = fmaf(a, S[i], dx * Bt[n]);
            acc = fmaf(S[i], Ct[n], acc);
          }
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0 && live) p.y[(long long)(first + t0 + t) * ((long long)p.H * P) + (long long)h * P + pcol] = fmaf(skip, x, acc);
    }
    __syncthreads();              // the buffer may be filled again
  }
  if (((p.mode == 0 && p.write_state) || p.mode == 1) && live) {
#pragma unroll
    for (int i = 0; i < NPER; ++i) {
      const int n = VEC ? ((i >> 2) * 32 + lane * 4 + (i & 3)) : (lane + SCAN_LANES * i);
      if (n < N) st[n] = S[i];
    }
  }
  if (p.mode == 1 && blockIdx.x == 0 && threadIdx.x == 0) *chunk_decay = decay_product;
}

// grid (ceil(H P N / 256), requests): a thread an entry of the state walks the request's chunks in order
__global__ void __launch_bounds__(256) ssm_chunk_states_kernel(float* __restrict__ chunk_state, const float* __restrict__ chunk_decay,
                                                               float* __restrict__ state, long long state_stride,
                                                               const int* __restrict__ state_slot, const int* __restrict__ row_start,
                                                               int H, int PN, int chunk_tokens, int max_chunks, int write_state) {
  const long long e = blockIdx.x * (long long)blockDim.x + threadIdx.x;
  const int b = blockIdx.y;
  const long long per = (long long)H * PN;
  if (e >= per) return;
  const int h = (int)(e / PN);
  const int chunks = ceil_div(row_start[b + 1] - row_start[b], chunk_tokens);
  if (chunks <= 0) return;
  float* slot = state + (long long)state_slot[b] * state_stride + e;
  float S = *slot;
  for (int c = 0; c < chunks; ++c) {
    float* at = chunk_state + ((long long)b * max_chunks + c) * per + e;
    const float last = *at;
    *at = S;
    S = fmaf(chunk_decay[((long long)b * max_chunks + c) * H + h], S, last);
  }
  if (write_state) *slot = S;
}

// grid (groups, rows): out[r, part] = w * v / rms(v), v = y * silu(z)
template <typename T>
__global__ void __launch_bounds__(256) gated_group_norm_kernel(const float* __restrict__ y, const float* __restrict__ z,
                                                               long long ld_z, const float* __restrict__ w, float eps,
                                                               T* __restrict__ out, int inner, int groups) {
  __shared__ float scratch[33];
  const int part = inner / groups;
  const int r = blockIdx.y, c0 = blockIdx.x * part;
  const float* yr = y + (long long)r * inner + c0;
  const float* zr = z + (long long)r * ld_z + c0;
  float ss = 0.f;
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float v = yr[c] * silu_f(zr[c]);
    ss += v * v;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)part + eps);
  for (int c = threadIdx.x; c < part; c += blockDim.x) {
    const float v = yr[c] * silu_f(zr[c]);
    out[(long long)r * inner + c0 + c] = from_f32<T>(v * inv * w[c0 + c]);
  }
}

}  // namespace tl

using namespace tl;

// in [rows, ld_in] (the C channels begin at in), taps [C, K], bias [C] or null, state: a slot's [K - 1, C] inputs begin at
// state + slot * state_stride; out [rows, ld_out]. act: 0 none, 1 SiLU.
extern "C" int tl_causal_conv_act(const float* in, long long ld_in, const float* taps, const float* bias, const float* state,
                                  long long state_stride, const int* state_slot, const int* req_of_row, const int* row_start,
                                  float* out, long long ld_out, int rows, int C, int K, int act, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && C > 0 && K >= 1 && K <= 64, "causal conv: %d rows, %d channels, %d taps", rows, C, K);
  TL_REQUIRE(rows <= 65535, "causal conv: %d rows in one launch; up to 65535", rows);
  TL_REQUIRE(act == TL_CONV_ACT_NONE || act == TL_CONV_ACT_SILU, "causal conv: activation %d", act);
  causal_conv_act_kernel<<<dim3(ceil_div(C, 256), rows), 256, 0, stream>>>(in, ld_in, taps, bias, state, state_stride, state_slot,
                                                                           req_of_row, row_start, out, ld_out, C, K, act);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_conv_state(const float* in, long long ld_in, float* state, long long state_stride, const int* state_slot,
                             const int* row_start, int requests, int C, int K, cudaStream_t stream) {
  if (requests == 0 || K <= 1) return 0;
  TL_REQUIRE(requests > 0 && requests <= 65535 && C > 0, "conv state: %d requests, %d channels", requests, C);
  conv_state_kernel<<<dim3(ceil_div(C, 256), requests), 256, 0, stream>>>(in, ld_in, state, state_stride, state_slot, row_start,
                                                                          C, K);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_ssm_scan(const float* xbc, long long ld_xbc, const float* dt, long long ld_dt, const float* dt_bias,
                           const float* a_log, const float* d_skip, float* state, long long state_stride,
                           const int* state_slot, const int* row_start, float* y, int requests, int H, int P, int N, int G,
                           int write_state, int chunk_tokens, int max_chunks, float* chunk_scratch, cudaStream_t stream) {
  if (requests == 0) return 0;
  TL_REQUIRE(requests > 0 && requests <= 65535 && H > 0 && H <= 65535 && P > 0 && N > 0 && G > 0 && H % G == 0,
             "ssm scan: %d requests, %d heads in %d groups, columns %d, state %d", requests, H, G, P, N);
  TL_REQUIRE(N <= SCAN_LANES * 32, "ssm scan: a state of %d rows; up to %d are implemented", N, SCAN_LANES * 32);
  ScanParams p;
  p.xbc = xbc; p.ld_xbc = ld_xbc; p.dt = dt; p.ld_dt = ld_dt; p.dt_bias = dt_bias; p.a_log = a_log; p.d_skip = d_skip;
  p.state = state; p.state_stride = state_stride; p.state_slot = state_slot; p.row_start = row_start; p.y = y;
  p.H = H; p.P = P; p.N = N; p.G = G; p.write_state = write_state;
  p.mode = 0; p.chunk_tokens = chunk_tokens; p.max_chunks = max_chunks; p.chunk_state = nullptr; p.chunk_decay = nullptr;
  const bool chunked = chunk_tokens > 0 && max_chunks > 1;
  TL_REQUIRE(!chunked || (chunk_scratch && (long long)requests * max_chunks <= 65535), "ssm scan: %d requests in %d chunks each",
             requests, max_chunks);
  if (chunked) {
    p.chunk_state = chunk_scratch;
    p.chunk_decay = chunk_scratch + (long long)requests * max_chunks * H * P * N;
  }
  const dim3 grid(ceil_div(P, SCAN_COLS), H, chunked ? requests * max_chunks : requests), block(SCAN_COLS * SCAN_LANES);
  const size_t smem = 2 * (size_t)(2 * SCAN_TOKENS * N + SCAN_TOKENS * SCAN_COLS + 3 * SCAN_TOKENS) * sizeof(float);
  const int per = ceil_div(N, SCAN_LANES);
  const bool vec = N % 4 == 0;
#define TL_SCAN(NPER_)                                                                    \
  do {                                                                                    \
    if (smem > 48 * 1024) {                                                               \
      cudaFuncSetAttribute(ssm_scan_kernel<(NPER_ < 4 ? 4 : NPER_), true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
      cudaFuncSetAttribute(ssm_scan_kernel<NPER_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
    }                                                                                     \
    if (vec) ssm_scan_kernel<(NPER_ < 4 ? 4 : NPER_), true><<<grid, block, smem, stream>>>(p); \
    else ssm_scan_kernel<NPER_, false><<<grid, block, smem, stream>>>(p);                 \
  } while (0)
#define TL_SCAN_ANY()              \
  do {                             \
    if (per <= 2) TL_SCAN(2);      \
    else if (per <= 4) TL_SCAN(4); \
    else if (per <= 8) TL_SCAN(8); \
    else if (per <= 16) TL_SCAN(16); \
    else TL_SCAN(32);              \
  } while (0)
  if (!chunked) {
    TL_SCAN_ANY();
    TL_LAUNCH_CHECK();
    return 0;
  }
  p.mode = 1;
  TL_SCAN_ANY();
  TL_LAUNCH_CHECK();
  ssm_chunk_states_kernel<<<dim3((unsigned)ceil_div64((long long)H * P * N, 256), requests), 256, 0, stream>>>(
      p.chunk_state, p.chunk_decay, state, state_stride, state_slot, row_start, H, P * N, chunk_tokens, max_chunks, write_state);
  TL_LAUNCH_CHECK();
  p.mode = 2;
  TL_SCAN_ANY();
#undef TL_SCAN_ANY
#undef TL_SCAN
  TL_LAUNCH_CHECK();
  return 0;
}

// Floats of scratch a chunked scan needs.
extern "C" long long tl_ssm_scan_scratch(int requests, int max_chunks, int H, int P, int N) {
  return (long long)requests * max_chunks * ((long long)H * P * N + H);
}

extern "C" int tl_gated_group_norm(const float* y, const float* z, long long ld_z, const float* w, float eps, void* out,
                                   int rows, int inner, int groups, int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && rows <= 65535 && inner > 0 && groups > 0 && inner % groups == 0,
             "gated group norm: %d rows of %d in %d parts", rows, inner, groups);
  const dim3 grid(groups, rows);
  if (dtype == TL_FP32) gated_group_norm_kernel<float><<<grid, 256, 0, stream>>>(y, z, ld_z, w, eps, (float*)out, inner, groups);
  else gated_group_norm_kernel<bf16><<<grid, 256, 0, stream>>>(y, z, ld_z, w, eps, (bf16*)out, inner, groups);
  TL_LAUNCH_CHECK();
  return 0;
}
