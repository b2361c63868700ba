// Layer norm (mean and variance, weight and bias) fused with the residual add; see LayerNormArgs in kernel_args.h.
// One block per output row; the row is kept in shared memory between the passes (sum, squared deviations, output),
// so the variance is the mean of the squared deviations from the mean and not a difference of two large sums.  The
// residual, every sum and both statistics are float32.
#include "common.cuh"
#include "kernel_args.h"

LLG_API const char* llg_last_error() { return g_llg_error; }

namespace {

template <typename OT, typename WT, bool VEC>
__global__ void add_layernorm_kernel(LayerNormArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float row[];
  __shared__ float red[32];
  const int j = blockIdx.x;
  const int r = a.rows ? a.rows[j] : j;
  const int hidden = a.hidden;
  float* res = a.residual + (long long)r * hidden;
  const bool any = a.branch[0] != nullptr;
  float sum = 0.f;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < hidden; i += blockDim.x * 4) {
      float4 v = *reinterpret_cast<const float4*>(res + i);
      if (any) {
        float4 t = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int b = 0; b < LLG_LN_BRANCHES; ++b) {
          if (!a.branch[b]) break;
          const float* p = a.branch[b] + (long long)r * hidden + i;
          for (int s = 0; s < a.n_partials[b]; ++s) {
            const float4 u = *reinterpret_cast<const float4*>(p + s * a.partial_stride);
            t.x += u.x; t.y += u.y; t.z += u.z; t.w += u.w;
          }
        }
        v.x = fmaf(a.scale, t.x, v.x); v.y = fmaf(a.scale, t.y, v.y);
        v.z = fmaf(a.scale, t.z, v.z); v.w = fmaf(a.scale, t.w, v.w);
        *reinterpret_cast<float4*>(res + i) = v;
      }
      *reinterpret_cast<float4*>(row + i) = v;
      sum += (v.x + v.y) + (v.z + v.w);
    }
  } else {
    for (int i = threadIdx.x; i < hidden; i += blockDim.x) {
      float v = res[i];
      if (any) {
        float t = 0.f;
#pragma unroll
        for (int b = 0; b < LLG_LN_BRANCHES; ++b) {
          if (!a.branch[b]) break;
          const float* p = a.branch[b] + (long long)r * hidden + i;
          for (int s = 0; s < a.n_partials[b]; ++s) t += p[s * a.partial_stride];
        }
        v = fmaf(a.scale, t, v);
        res[i] = v;
      }
      row[i] = v;
      sum += v;
    }
  }
  const float mean = block_sum(sum, red) / (float)hidden;
  float dev = 0.f;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x) {      // block_sum's barriers stand between the writes of row and here
    const float d = row[i] - mean;
    dev += d * d;
  }
  const float inv = 1.0f / sqrtf(block_sum(dev, red) / (float)hidden + a.eps);
  const WT* w = (const WT*)a.weight;
  const WT* bs = (const WT*)a.bias;
  OT* o = (OT*)a.out + (long long)j * hidden;
  for (int i = threadIdx.x; i < hidden; i += blockDim.x)
    o[i] = from_f32<OT>((row[i] - mean) * inv * to_f32(w[i]) + to_f32(bs[i]));
}

}  // namespace

LLG_API int llg_add_layernorm(const LayerNormArgs* args, cudaStream_t stream) {
  const LayerNormArgs& a = *args;
  LLG_REQUIRE(a.n_out >= 0 && a.hidden > 0, "add_layernorm: bad sizes n_out=%d hidden=%d", a.n_out, a.hidden);
  LLG_REQUIRE(a.eps > 0.f, "add_layernorm: eps must be positive");
  for (int b = 0; b < LLG_LN_BRANCHES; ++b) {
    LLG_REQUIRE(!a.branch[b] || a.n_partials[b] >= 1, "add_layernorm: a set of partials needs at least one");
    LLG_REQUIRE(!a.branch[b] || b == 0 || a.branch[b - 1], "add_layernorm: sets of partials must be given in order");
  }
  if (a.n_out == 0) return 0;
  bool vec = a.hidden % 4 == 0 && a.partial_stride % 4 == 0 && ((uintptr_t)a.residual % 16) == 0;
  for (int b = 0; b < LLG_LN_BRANCHES; ++b) vec = vec && ((uintptr_t)a.branch[b] % 16) == 0;
  const int threads = a.hidden >= 4096 ? 512 : (a.hidden >= 1024 ? 256 : 128);
  const size_t smem = (size_t)a.hidden * sizeof(float);
  LLG_REQUIRE(smem <= 200 * 1024, "add_layernorm: rows of %d elements do not fit shared memory", a.hidden);
#define LAUNCH(OT, WT)                                                                                          \
  do {                                                                                                          \
    auto k = vec ? add_layernorm_kernel<OT, WT, true> : add_layernorm_kernel<OT, WT, false>;                    \
    if (smem > 48 * 1024) {                                                                                     \
      cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);          \
      if (e != cudaSuccess) return llg_fail("add_layernorm: shared memory %zu: %s", smem, cudaGetErrorString(e)); \
    }                                                                                                           \
    llg_launch(k, dim3(a.n_out), dim3(threads), smem, stream, a);                                               \
  } while (0)
  if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_F32) LAUNCH(float, float);
  else if (a.out_dtype == LLG_F32 && a.w_dtype == LLG_BF16) LAUNCH(float, __nv_bfloat16);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_F32) LAUNCH(__nv_bfloat16, float);
  else if (a.out_dtype == LLG_BF16 && a.w_dtype == LLG_BF16) LAUNCH(__nv_bfloat16, __nv_bfloat16);
  else return llg_fail("add_layernorm: unknown dtypes out=%d weight=%d", a.out_dtype, a.w_dtype);
#undef LAUNCH
  return llg_check_launch("add_layernorm");
}
