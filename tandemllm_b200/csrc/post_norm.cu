// A norm behind a branch (the second norm of a layer whose sublayers are normed before and after), fused with the
// residual add, and a vector added to every row of the residual stream.
//
//   d[r] = (sum of the dense parts)[r] * (gate ? sigmoid(gate[r]) : 1) + sum_j wts[r, j] * expert_rows[pos_of_pair[r k + j]]
//   residual[r] += weight * d[r] * rsqrt(mean(d[r]^2) + eps)
//   with `pre_weight`: normed[i] = pre_weight * residual[r] * rsqrt(mean(residual[r]^2) + eps)  (the norm in front of the next
//   sublayer in the same pass; with `gather`, output row i reads row gather[i] and the residual stays as it was)
//
// The branch output comes in the forms the products leave it in: a 32-bit tensor or partial sums of a product split along
// k (added in order), the rows of a routed expert layer (weighed and added in ascending expert id), or both (a shared
// feed-forward beside the routed one, times a gate a row). Everything is 32-bit; one block a row, fixed orders of addition.
#include "route.cuh"

namespace tl {

struct PostNormParams {
  float* residual;
  const float* delta;
  int parts;
  long long part_stride;
  const float* delta_gate;   // [rows] logits or nullptr: the dense parts times sigmoid(logit)
  const float* expert_rows;
  int expert_parts;
  long long expert_part_stride;
  const int* pos_of_pair;
  const int* ids;
  const float* wts;
  int top_k;
  const float* weight;
  float eps;
  int hidden;
  const float* pre_weight;   // the next norm's weight, or nullptr: only the add
  float pre_eps;
  void* normed;
  const int* gather;
  int few_rows;              // a step of few rows (few blocks): the form whose loads of a source are all in flight together
};

// FEW: the form for a step of few rows (see `few_rows`), a kernel of its own so that the other keeps its few registers.
template <typename T, bool FEW>
__global__ void __launch_bounds__(256) add_normed_kernel(PostNormParams p) {
  extern __shared__ __align__(16) float row[];          // hidden floats, then 33 for the reductions
  float* scratch = row + p.hidden;
  __shared__ int s_src[MAX_TOP_K];
  __shared__ float s_w[MAX_TOP_K];
  const int hidden = p.hidden;
  const int r = p.gather ? p.gather[blockIdx.x] : (int)blockIdx.x;
  if (p.expert_rows) {
    if (threadIdx.x < 32) {
      // the row's slots in ascending expert id (the slot index breaks ties)
      const int k = p.top_k, j = threadIdx.x;
      const bool mine = j < k;
      const int e = mine ? p.ids[(long long)r * k + j] : 0x7fffffff;
      const int src = mine ? p.pos_of_pair[(long long)r * k + j] : 0;
      const float w = mine ? p.wts[(long long)r * k + j] : 0.f;
      int rank = 0;
      for (int i = 0; i < k; ++i) {
        const int ei = __shfl_sync(0xffffffffu, e, i);
        rank += (ei < e) || (ei == e && i < j);
      }
      if (mine) {
        s_src[rank] = src;
        s_w[rank] = w;
      }
    }
    __syncthreads();
  }
  const float g = p.delta_gate ? 1.f / (1.f + expf(-p.delta_gate[r])) : 1.f;
  float ss = 0.f;
  constexpr int CPT = 16;           // columns a thread holds in registers in the form for rows of up to 16 x 256 numbers
  if (FEW && hidden <= CPT * (int)blockDim.x) {
    // Source by source, a thread's loads of one source all sent before the first is used: a decode step has a handful of
    // blocks, and their time is the chain of round trips to L2, one a source instead of one a source and column.
    float d[CPT], routed[CPT];
#pragma unroll
    for (int i = 0; i < CPT; ++i) d[i] = routed[i] = 0.f;
    if (p.delta) {
      for (int s = 0; s < p.parts; ++s) {
        const float* src = p.delta + (long long)s * p.part_stride + (size_t)r * hidden;
#pragma unroll
        for (int i = 0; i < CPT; ++i) {
          const int c = threadIdx.x + i * blockDim.x;
          if (c < hidden) d[i] += src[c];
        }
      }
#pragma unroll
      for (int i = 0; i < CPT; ++i) d[i] *= g;
    }
    if (p.expert_rows) {
      for (int j = 0; j < p.top_k; ++j) {
        float v[CPT];
#pragma unroll
        for (int i = 0; i < CPT; ++i) v[i] = 0.f;
        for (int s = 0; s < p.expert_parts; ++s) {
          const float* src = p.expert_rows + (long long)s * p.expert_part_stride + (long long)s_src[j] * hidden;
#pragma unroll
          for (int i = 0; i < CPT; ++i) {
            const int c = threadIdx.x + i * blockDim.x;
            if (c < hidden) v[i] += src[c];
          }
        }
#pragma unroll
        for (int i = 0; i < CPT; ++i) routed[i] = fmaf(s_w[j], v[i], routed[i]);
      }
#pragma unroll
      for (int i = 0; i < CPT; ++i) d[i] = routed[i] + d[i];
    }
#pragma unroll
    for (int i = 0; i < CPT; ++i) {
      const int c = threadIdx.x + i * blockDim.x;
      if (c < hidden) {
        row[c] = d[i];
        ss += d[i] * d[i];
      }
    }
  } else
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    float d = 0.f;
    if (p.delta) {
      for (int s = 0; s < p.parts; ++s) d += p.delta[(long long)s * p.part_stride + (size_t)r * hidden + c];
      d *= g;
    }
    if (p.expert_rows) {
      float routed = 0.f;
      for (int j = 0; j < p.top_k; ++j) {
        float v = 0.f;
        for (int s = 0; s < p.expert_parts; ++s)
          v += p.expert_rows[(long long)s * p.expert_part_stride + (long long)s_src[j] * hidden + c];
        routed = fmaf(s_w[j], v, routed);
      }
      d = routed + d;
    }
    row[c] = d;
    ss += d * d;
  }
  ss = block_sum(ss, scratch);
  const float inv = rsqrtf(ss / (float)hidden + p.eps);
  float* res = p.residual + (size_t)r * hidden;
  float ss2 = 0.f;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) {
    const float x = res[c] + row[c] * inv * p.weight[c];
    if (!p.gather) res[c] = x;
    row[c] = x;
    ss2 += x * x;
  }
  if (!p.pre_weight) return;
  ss2 = block_sum(ss2, scratch);
  const float inv2 = rsqrtf(ss2 / (float)hidden + p.pre_eps);
  T* out = reinterpret_cast<T*>(p.normed) + (size_t)blockIdx.x * hidden;
  for (int c = threadIdx.x; c < hidden; c += blockDim.x) out[c] = from_f32<T>(row[c] * inv2 * p.pre_weight[c]);
}

// out[r] = x[r, :] . w: a warp a row (a projection onto one number a row, such as the logit of a gate)
template <typename T>
__global__ void __launch_bounds__(256) row_dot_kernel(const T* __restrict__ x, long long ld_x, const T* __restrict__ w,
                                                      float* __restrict__ out, int rows, int hidden) {
  const int r = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
  if (r >= rows) return;
  const T* xr = x + (long long)r * ld_x;
  float acc = 0.f;
#pragma unroll 8
  for (int c = lane; c < hidden; c += 32) acc = fmaf(to_f32(xr[c]), to_f32(w[c]), acc);
  acc = warp_sum(acc);
  if (lane == 0) out[r] = acc;
}

// residual[r, :] += vec
__global__ void add_vector_kernel(float* __restrict__ residual, const float* __restrict__ vec, long long n, int hidden) {
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
    residual[i] += vec[i % hidden];
}

}  // namespace tl

using namespace tl;

extern "C" int tl_add_normed(float* residual, const float* delta, int parts, long long part_stride, const float* delta_gate,
                             const float* expert_rows, int expert_parts, long long expert_part_stride, const int* pos_of_pair,
                             const int* ids, const float* wts, int top_k, const float* weight, float eps,
                             const float* pre_weight, float pre_eps, void* normed, const int* gather, int rows, int hidden,
                             int dtype, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && hidden <= 16384, "add_normed: %d rows of %d", rows, hidden);
  TL_REQUIRE(residual && weight && (delta || expert_rows), "add_normed: a residual, a weight and a branch output are needed");
  TL_REQUIRE(!delta || parts >= 1, "add_normed: %d parts", parts);
  TL_REQUIRE(!expert_rows || (pos_of_pair && ids && wts && top_k > 0 && top_k <= MAX_TOP_K && expert_parts >= 1),
             "add_normed: expert rows with top-%d in %d parts", top_k, expert_parts);
  TL_REQUIRE(!pre_weight || normed, "add_normed: the following norm needs a place for its rows");
  TL_REQUIRE(!gather || pre_weight, "add_normed: chosen rows are only read for the following norm");
  PostNormParams p;
  p.residual = residual; p.delta = delta; p.parts = parts; p.part_stride = part_stride; p.delta_gate = delta_gate;
  p.expert_rows = expert_rows; p.expert_parts = expert_parts; p.expert_part_stride = expert_part_stride;
  p.pos_of_pair = pos_of_pair; p.ids = ids; p.wts = wts; p.top_k = top_k; p.weight = weight; p.eps = eps; p.hidden = hidden;
  p.pre_weight = pre_weight; p.pre_eps = pre_eps; p.normed = normed; p.gather = gather;
  p.few_rows = rows <= 2 * sm_count() ? 1 : 0;
  const size_t smem = (size_t)(hidden + 33) * sizeof(float);
#define TL_ADD_NORMED(T_, FEW_)                                                                                         \
  do {                                                                                                                  \
    if (smem > 48 * 1024)                                                                                               \
      cudaFuncSetAttribute(add_normed_kernel<T_, FEW_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);        \
    add_normed_kernel<T_, FEW_><<<rows, 256, smem, stream>>>(p);                                                        \
  } while (0)
  if (dtype == TL_FP32) {
    if (p.few_rows) TL_ADD_NORMED(float, true);
    else TL_ADD_NORMED(float, false);
  } else {
    if (p.few_rows) TL_ADD_NORMED(bf16, true);
    else TL_ADD_NORMED(bf16, false);
  }
#undef TL_ADD_NORMED
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_row_dot(const void* x, long long ld_x, const void* w, float* out, int rows, int hidden, int dtype,
                          cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && x && w && out, "row dot: %d rows of %d", rows, hidden);
  if (dtype == TL_FP32) row_dot_kernel<float><<<ceil_div(rows, 8), 256, 0, stream>>>((const float*)x, ld_x, (const float*)w, out, rows, hidden);
  else row_dot_kernel<bf16><<<ceil_div(rows, 8), 256, 0, stream>>>((const bf16*)x, ld_x, (const bf16*)w, out, rows, hidden);
  TL_LAUNCH_CHECK();
  return 0;
}

extern "C" int tl_add_vector(float* residual, const float* vec, int rows, int hidden, cudaStream_t stream) {
  if (rows == 0) return 0;
  TL_REQUIRE(rows > 0 && hidden > 0 && residual && vec, "add_vector: %d rows of %d", rows, hidden);
  const long long n = (long long)rows * hidden;
  const long long most = (long long)sm_count() * 8;
  const int blocks = (int)(ceil_div64(n, 256) < most ? ceil_div64(n, 256) : most);
  add_vector_kernel<<<blocks, 256, 0, stream>>>(residual, vec, n, hidden);
  TL_LAUNCH_CHECK();
  return 0;
}
