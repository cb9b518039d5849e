// Argument block and epilogue shared by the projection kernels.
#pragma once
#include "common.cuh"

namespace mlora {

// Residual add + RMSNorm folded into two neighbouring decode-size projections (tensor-core kernel, T <= 32):
//   producer (res != nullptr):   res[t, o] += y[t, o];  y[t, o] = bf16(res[t, o] * norm_w[o])  -- the row's 1/rms is NOT
//                                applied; sumsq_out[row_tile * 32 + t] = sum over the tile's 128 outputs of res[t, o]^2
//   consumer (sumsq_in != nullptr): y[t, :] *= rsqrt(sum_j sumsq_in[j * 32 + t] / norm_dim + eps)  before the activation,
//                                i.e. the 1/rms of its input rows, which is a per-row factor of a linear map.
struct NormFuse {
  float* res;
  int64_t ld_res;
  const bf16* norm_w;
  float* sumsq_out;
  const float* sumsq_in;
  int n_sumsq_in;
  float eps;
  int norm_dim;
};

struct LinearArgs {
  const bf16* x;
  int64_t ldx;
  const bf16* W;
  void* y;
  int64_t ldy;
  int T, in, out;
  const float* u;        // [T, n_mod*r_max] or nullptr
  const bf16* B_all;     // [N, out, r_max]
  const int32_t* ranks;  // [N]
  const float* scales;   // [N]
  const int32_t* slots;  // [T]
  int r_max, n_mod;      // B row pitch / u slice width, number of u slices per row
  int mod_off[9];
  int flags;
  int n_adapters;        // slots >= n_adapters are treated as "no adapter"
  int full_rank;         // 1: every row uses all r_max entries (zero-padded), ranks[] is ignored
  const float* y_in;     // per-row expand with MLORA_SILU_MUL: the projection's pre-activations, fp32 [T, out]
  NormFuse nf;           // all zero: plain projection
};

// Module (q/k/v, gate/up ...) that owns output row o.
__device__ __forceinline__ int module_of(const LinearArgs& a, int o) {
  int m = 0;
#pragma unroll 1
  while (m + 1 < a.n_mod && o >= a.mod_off[m + 1]) ++m;
  return m;
}

// scale[s] * sum_j u[t, m*r_max + j] * B_all[s, o, j]   (0 when the row has no adapter)
__device__ __forceinline__ float lora_expand(const LinearArgs& a, int t, int o) {
  if (a.u == nullptr) return 0.f;
  const int s = a.slots[t];
  if (s < 0 || s >= a.n_adapters) return 0.f;
  const int r = a.full_rank ? a.r_max : a.ranks[s];
  const int m = module_of(a, o);
  const float* ur = a.u + (size_t)t * (a.r_max * a.n_mod) + m * a.r_max;
  const bf16* b = a.B_all + ((size_t)s * a.out + o) * a.r_max;
  float acc = 0.f;
  if ((a.r_max & 7) == 0) {
    for (int j = 0; j < r; j += 8) {
      float bf[8];
      unpack8(ld_cached(b + j), bf);
#pragma unroll
      for (int e = 0; e < 8; ++e)
        if (j + e < r) acc = fmaf(ur[j + e], bf[e], acc);
    }
  } else {
    for (int j = 0; j < r; ++j) acc = fmaf(ur[j], __bfloat162float(b[j]), acc);
  }
  return a.scales[s] * acc;
}

// (fast division: two instructions instead of a subroutine -- the epilogue that calls this 32 times per thread
// runs once per tile, from cold instruction caches)
__device__ __forceinline__ float silu_mul(float g, float up) { return __fdividef(g, 1.f + __expf(-g)) * up; }

__device__ __forceinline__ void store_out(const LinearArgs& a, int t, int col, float v) {
  if (a.flags & MLORA_OUT_F32)
    reinterpret_cast<float*>(a.y)[(size_t)t * a.ldy + col] = v;
  else
    reinterpret_cast<bf16*>(a.y)[(size_t)t * a.ldy + col] = __float2bfloat16_rn(v);
}

int launch_linear_simt(const LinearArgs& a, cudaStream_t st);
// Tensor-core (tcgen05) weight-streaming kernel; returns MLORA_OK or an error.
bool linear_tc_supported(const LinearArgs& a);
size_t linear_tc_workspace(int T, int in, int out);
void linear_tc_plan(int T, int in, int out, int32_t* v12);
int launch_linear_tc(const LinearArgs& a, void* work, size_t work_bytes, cudaStream_t st);
// LoRA expand laid out by (row, output feature), added to y in place (batches with many distinct adapters).
bool lora_expand_rows_supported(const LinearArgs& a);
bool lora_expand_silu_supported(const LinearArgs& a);  // the same expand in front of the SiLU*up of interleaved gate/up rows
int launch_lora_expand_rows(const LinearArgs& a, cudaStream_t st);
// LoRA shrink as a segmented grouped GEMM on the tensor cores (prefill sizes).
bool lora_shrink_tc_supported(const void* x, int64_t ldx, const void* A_all, const float* u, int T, int in, int r_tot);
int launch_lora_shrink_tc(const void* x, int64_t ldx, const void* A_all, const int32_t* slots, int n_adapters, int T,
                          int in, int r_tot, float* u, cudaStream_t st);
size_t packed_weight_bytes(int out, int in);
size_t packed_lora_b_bytes(int n_adapters, int out, int r_max);
int launch_pack_lora_b(const void* B, int n_adapters, int out, int r_max, void* Bp, cudaStream_t st);
int launch_pack_weight(const void* W, int out, int in, void* Wp, cudaStream_t st);

}  // namespace mlora
