// Row-wise kernels of the decode step: fused residual add + RMSNorm, embedding gather, greedy
// argmax, and the device-side sequence-length bookkeeping.  One CTA per row, 128-bit accesses,
// warp-shuffle reductions.
#include <cfloat>

#include "common.cuh"

namespace mlora {
namespace {

__device__ __forceinline__ float block_sum(float v, float* sm /*[33]*/) {
  v = warp_sum(v);
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) sm[w] = v;
  __syncthreads();
  if (w == 0) {
    float t = lane < (blockDim.x + 31) / 32 ? sm[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) sm[32] = t;
  }
  __syncthreads();
  float r = sm[32];
  __syncthreads();
  return r;
}

// res += delta; out = res * rsqrt(mean(res^2) + eps) * w.  H % 8 == 0.  The row is kept in
// registers between the two passes (up to 4 chunks of 8 per thread = H <= 8192 at 256 threads),
// longer rows re-read the updated residual.
constexpr int kNormThreads = 256;
constexpr int kNormChunks = 4;

__global__ void __launch_bounds__(kNormThreads) residual_rmsnorm_kernel(const bf16* __restrict__ delta,
                                                                        float* __restrict__ res,
                                                                        const bf16* __restrict__ w, float eps,
                                                                        bf16* __restrict__ out, int H) {
  __shared__ float sm[33];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  float* r = res + row * H;
  const bf16* d = delta ? delta + row * H : nullptr;
  float keep[kNormChunks][8];
  float ss = 0.f;
  // pass 1: add the delta, store the new residual, accumulate the sum of squares.  The loads of all of a
  // thread's chunks are issued before the first store (the stores go to the array the loads read, so the
  // compiler keeps their order): one round trip for the row instead of one per chunk.
  auto add_store = [&](int k, const float4& a, const float4& b, const uint4& draw, float (&v)[8]) {
    v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
    if (d) {
      float df[8];
      unpack8(draw, df);
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] += df[i];
      *reinterpret_cast<float4*>(r + k) = make_float4(v[0], v[1], v[2], v[3]);
      *reinterpret_cast<float4*>(r + k + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
  };
  {
    float4 ra[kNormChunks], rb[kNormChunks];
    uint4 rd[kNormChunks];
#pragma unroll
    for (int c = 0; c < kNormChunks; ++c) {
      const int k = (c * kNormThreads + threadIdx.x) * 8;
      if (k < H) {
        ra[c] = *reinterpret_cast<const float4*>(r + k);
        rb[c] = *reinterpret_cast<const float4*>(r + k + 4);
        if (d) rd[c] = ld_cached(d + k);
      }
    }
#pragma unroll
    for (int c = 0; c < kNormChunks; ++c) {
      const int k = (c * kNormThreads + threadIdx.x) * 8;
      if (k < H) add_store(k, ra[c], rb[c], rd[c], keep[c]);
    }
  }
  for (int k = (kNormChunks * kNormThreads + threadIdx.x) * 8; k < H; k += kNormThreads * 8) {
    float v[8];
    const float4 a = *reinterpret_cast<const float4*>(r + k), b = *reinterpret_cast<const float4*>(r + k + 4);
    uint4 dr = make_uint4(0u, 0u, 0u, 0u);
    if (d) dr = ld_cached(d + k);
    add_store(k, a, b, dr, v);
  }
  uint4 wq[kNormChunks];  // norm weights: requested before the block-wide reduction, used after it
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int k = (c * kNormThreads + threadIdx.x) * 8;
    if (k < H) wq[c] = ld_cached(w + k);
  }
  ss = block_sum(ss, sm);
  const float inv = rsqrtf(ss / (float)H + eps);
  // pass 2: scale and write
  auto write = [&](int k, const float (&v)[8], const uint4& wraw) {
    float wf[8], o[8];
    unpack8(wraw, wf);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = v[i] * inv * wf[i];
    *reinterpret_cast<uint4*>(out + row * H + k) = pack8(o);
  };
#pragma unroll
  for (int c = 0; c < kNormChunks; ++c) {
    const int k = (c * kNormThreads + threadIdx.x) * 8;
    if (k < H) write(k, keep[c], wq[c]);
  }
  for (int k = (kNormChunks * kNormThreads + threadIdx.x) * 8; k < H; k += kNormThreads * 8) {
    float4 a = *reinterpret_cast<const float4*>(r + k);
    float4 b = *reinterpret_cast<const float4*>(r + k + 4);
    float v[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
    write(k, v, ld_cached(w + k));
  }
}

// ---- fused residual add + RMSNorm + LoRA shrink ---------------------------------------------------------------
// The q/k/v (or gate/up) shrink reads exactly the row this kernel has just normalised, and both kernels are chains
// of a few memory round trips with a launch in between.  Fused, every thread keeps its elements of the normalised
// row in registers and multiplies them with the same positions of a group of A rows, all requested in ONE round
// trip while the row statistics are still being reduced; the per-row dot products are then block-wide sums.
// kNsSplit CTAs share a token row: each recomputes the (cheap) normalisation and takes a quarter of the rank
// rows, so a CTA stays small -- and uses no shared memory to speak of -- and the projection launched behind it
// can become resident beside it.  Only split 0 writes the residual and the normalised row; because the other
// splits read the OLD residual while it does, the residual goes from res_in to a different buffer res_out.
constexpr int kNsThreads = 256;
constexpr int kNsSplit = 4;
constexpr int kNsMaxH = 8192;

template <int NCH>  // chunks of 8 per thread: 2 (H <= 4096) or 4 (H <= 8192)
__global__ void __launch_bounds__(kNsThreads) rmsnorm_shrink_kernel(const bf16* __restrict__ delta,
                                                                    const float* __restrict__ res_in,
                                                                    float* __restrict__ res_out,
                                                                    const bf16* __restrict__ w, float eps,
                                                                    bf16* __restrict__ out, int H,
                                                                    const bf16* __restrict__ A_all,
                                                                    const int32_t* __restrict__ slots, int n_adapters,
                                                                    int r_tot, float* __restrict__ u) {
  constexpr int GROUP = 24 / NCH;  // A rows requested together: 24 128-bit loads in flight per thread
  __shared__ float sm[33];
  __shared__ float sred[kNsThreads / 32][GROUP];
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.y;
  const int split = blockIdx.x;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int slot = slots[row];
  const bool has = slot >= 0 && slot < n_adapters;
  const int per = (r_tot + kNsSplit - 1) / kNsSplit;
  const int j0 = split * per, j1 = min(r_tot, j0 + per);  // rank rows of this CTA
  const float* r = res_in + row * H;
  const bf16* d = delta ? delta + row * H : nullptr;
  // ---- residual add, sum of squares (every split) ----
  float keep[NCH][8];
  float ss = 0.f;
  {
    float4 ra[NCH], rb[NCH];
    uint4 rd[NCH];
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int k = (c * kNsThreads + threadIdx.x) * 8;
      if (k < H) {
        ra[c] = *reinterpret_cast<const float4*>(r + k);
        rb[c] = *reinterpret_cast<const float4*>(r + k + 4);
        if (d) rd[c] = ld_cached(d + k);
      }
    }
#pragma unroll
    for (int c = 0; c < NCH; ++c) {
      const int k = (c * kNsThreads + threadIdx.x) * 8;
      float (&v)[8] = keep[c];
#pragma unroll
      for (int i = 0; i < 8; ++i) v[i] = 0.f;
      if (k < H) {
        v[0] = ra[c].x, v[1] = ra[c].y, v[2] = ra[c].z, v[3] = ra[c].w;
        v[4] = rb[c].x, v[5] = rb[c].y, v[6] = rb[c].z, v[7] = rb[c].w;
        if (d) {
          float df[8];
          unpack8(rd[c], df);
#pragma unroll
          for (int i = 0; i < 8; ++i) v[i] += df[i];
        }
        if (split == 0) {
          *reinterpret_cast<float4*>(res_out + row * H + k) = make_float4(v[0], v[1], v[2], v[3]);
          *reinterpret_cast<float4*>(res_out + row * H + k + 4) = make_float4(v[4], v[5], v[6], v[7]);
        }
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
      }
    }
  }
  uint4 wq[NCH];
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = (c * kNsThreads + threadIdx.x) * 8;
    if (k < H) wq[c] = ld_cached(w + k);
  }
  // A rows of the first group: requested before the block-wide reduction
  uint4 av[GROUP][NCH];
  auto request = [&](int jb) {
#pragma unroll
    for (int jj = 0; jj < GROUP; ++jj) {
      if (jb + jj < j1) {
        const bf16* a = A_all + ((size_t)slot * r_tot + jb + jj) * H;
#pragma unroll
        for (int c = 0; c < NCH; ++c) {
          const int k = (c * kNsThreads + threadIdx.x) * 8;
          if (k < H) av[jj][c] = ld_cached(a + k);
        }
      }
    }
  };
  if (has) request(j0);
  ss = block_sum(ss, sm);
  const float inv = rsqrtf(ss / (float)H + eps);
  // ---- normalised row: written by split 0, kept (as rounded to bf16) by everyone ----
#pragma unroll
  for (int c = 0; c < NCH; ++c) {
    const int k = (c * kNsThreads + threadIdx.x) * 8;
    if (k < H) {
      float wf[8], o[8];
      unpack8(wq[c], wf);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] = keep[c][i] * inv * wf[i];
      const uint4 packed = pack8(o);
      if (split == 0) *reinterpret_cast<uint4*>(out + row * H + k) = packed;
      unpack8(packed, keep[c]);  // exactly what the projection (and a separate shrink) would read
    }
  }
  // ---- shrink: u[row, j] = A[slot, j, :] . xn ----
  for (int jb = j0; jb < j1; jb += GROUP) {
    float part[GROUP];
    if (has) {
      if (jb != j0) request(jb);
#pragma unroll
      for (int jj = 0; jj < GROUP; ++jj) {
        float acc = 0.f;
        if (jb + jj < j1) {
#pragma unroll
          for (int c = 0; c < NCH; ++c) {
            if ((c * kNsThreads + (int)threadIdx.x) * 8 < H) {
              float af[8];
              unpack8(av[jj][c], af);
#pragma unroll
              for (int i = 0; i < 8; ++i) acc = fmaf(af[i], keep[c][i], acc);
            }
          }
        }
        part[jj] = warp_sum(acc);
      }
      if (lane == 0) {
#pragma unroll
        for (int jj = 0; jj < GROUP; ++jj) sred[warp][jj] = part[jj];
      }
    }
    __syncthreads();
    if (threadIdx.x < GROUP && jb + (int)threadIdx.x < j1) {
      float acc = 0.f;
      if (has) {
#pragma unroll
        for (int wv = 0; wv < kNsThreads / 32; ++wv) acc += sred[wv][threadIdx.x];
      }
      u[row * r_tot + jb + threadIdx.x] = acc;
    }
    __syncthreads();
  }
}

__global__ void __launch_bounds__(256) embed_kernel(const int32_t* __restrict__ ids, const bf16* __restrict__ E,
                                                    int H, int vocab, float* __restrict__ res,
                                                    bf16* __restrict__ out_bf16) {
  pdl_launch_dependents();
  pdl_wait();
  const size_t row = blockIdx.x;
  int id = ids[row];
  id = min(max(id, 0), vocab - 1);  // out-of-range ids are clamped, never dereferenced
  const bf16* e = E + (size_t)id * H;
  for (int k = threadIdx.x * 8; k < H; k += blockDim.x * 8) {
    uint4 raw = ld_cached(e + k);
    if (res) {
      float f[8];
      unpack8(raw, f);
      *reinterpret_cast<float4*>(res + row * H + k) = make_float4(f[0], f[1], f[2], f[3]);
      *reinterpret_cast<float4*>(res + row * H + k + 4) = make_float4(f[4], f[5], f[6], f[7]);
    }
    if (out_bf16) *reinterpret_cast<uint4*>(out_bf16 + row * H + k) = raw;
  }
}

// First index of the maximum (numpy argmax semantics; NaN never wins).
__global__ void __launch_bounds__(1024) argmax_kernel(const float* __restrict__ logits, int64_t ld, int V,
                                                      int32_t* __restrict__ tok) {
  __shared__ float sv[32];
  __shared__ int si[32];
  pdl_launch_dependents();
  pdl_wait();
  const float* l = logits + (size_t)blockIdx.x * ld;
  float best = -FLT_MAX;
  int bi = 0x7fffffff;
  auto take = [&](float v, int i) {  // maximum, lowest index on ties (any visiting order)
    if (v > best || (v == best && i < bi)) {
      best = v;
      bi = i;
    }
  };
  // 128-bit loads, four per thread in flight: a row is 128 KB read by one CTA, i.e. a chain of L2 round trips
  const int V4 = ((reinterpret_cast<uintptr_t>(l) & 15) == 0) ? V / 4 : 0;
  const float4* l4 = reinterpret_cast<const float4*>(l);
  for (int i = threadIdx.x; i < V4; i += blockDim.x * 4) {
    float4 q[4];
#pragma unroll
    for (int u = 0; u < 4; ++u)
      if (i + u * (int)blockDim.x < V4) q[u] = l4[i + u * blockDim.x];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int idx = i + u * (int)blockDim.x;
      if (idx < V4) {
        take(q[u].x, 4 * idx);
        take(q[u].y, 4 * idx + 1);
        take(q[u].z, 4 * idx + 2);
        take(q[u].w, 4 * idx + 3);
      }
    }
  }
  for (int i = 4 * V4 + threadIdx.x; i < V; i += blockDim.x) take(l[i], i);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    float ov = __shfl_xor_sync(0xffffffffu, best, o);
    int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ov > best || (ov == best && oi < bi)) {
      best = ov;
      bi = oi;
    }
  }
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) {
    sv[w] = best;
    si[w] = bi;
  }
  __syncthreads();
  if (w == 0) {
    best = lane < (blockDim.x >> 5) ? sv[lane] : -FLT_MAX;
    bi = lane < (blockDim.x >> 5) ? si[lane] : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      float ov = __shfl_xor_sync(0xffffffffu, best, o);
      int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ov > best || (ov == best && oi < bi)) {
        best = ov;
        bi = oi;
      }
    }
    if (lane == 0) tok[blockIdx.x] = bi == 0x7fffffff ? 0 : bi;
  }
}

__global__ void kv_begin_decode_kernel(const int32_t* __restrict__ row_slot, int32_t* __restrict__ seq_lens,
                                       int32_t* __restrict__ row_pos, int B) {
  pdl_launch_dependents();
  pdl_wait();
  int b = blockIdx.x * blockDim.x + threadIdx.x;
  if (b < B) {
    int s = row_slot[b];
    int p = seq_lens[s];
    row_pos[b] = p;
    seq_lens[s] = p + 1;  // one row per sequence in a decode step, so no two threads share s
  }
}

}  // namespace
}  // namespace mlora

using namespace mlora;

extern "C" int mlora_residual_rmsnorm(const void* d_delta, float* d_res, const void* d_w, float eps, void* d_out,
                                      int32_t T, int32_t H, void* stream) {
  MLORA_REQUIRE(T >= 0 && H > 0 && H % 8 == 0, "residual_rmsnorm: H must be a positive multiple of 8 (H=%d)", H);
  MLORA_REQUIRE(d_res && d_w && d_out, "residual_rmsnorm: null pointer");
  MLORA_REQUIRE(aligned16(d_res) && aligned16(d_w) && aligned16(d_out) && aligned16(d_delta),
                "residual_rmsnorm: pointers must be 16-byte aligned");
  if (T == 0) return MLORA_OK;
  launch_pdl_if(pdl_enabled_norm(), residual_rmsnorm_kernel, T, kNormThreads, 0, (cudaStream_t)stream, (const bf16*)d_delta, d_res,
             (const bf16*)d_w, eps, (bf16*)d_out, H);
  count_launch();
  MLORA_CHECK_LAUNCH("residual_rmsnorm_kernel");
  return MLORA_OK;
}

extern "C" int mlora_residual_rmsnorm_shrink(const void* d_delta, const float* d_res_in, float* d_res_out, const void* d_w,
                                             float eps, void* d_out, int32_t T, int32_t H, const void* d_A_all,
                                             const int32_t* d_slots, int32_t n_adapters, int32_t r_tot, float* d_u,
                                             void* stream) {
  MLORA_REQUIRE(T >= 0 && H > 0 && H % 8 == 0 && H <= kNsMaxH, "residual_rmsnorm_shrink: H must be a multiple of 8 up to %d (H=%d)",
                kNsMaxH, H);
  MLORA_REQUIRE(d_res_in && d_res_out && d_w && d_out && d_A_all && d_slots && d_u, "residual_rmsnorm_shrink: null pointer");
  MLORA_REQUIRE((const void*)d_res_in != (const void*)d_res_out, "residual_rmsnorm_shrink: res_in and res_out must be different buffers");
  MLORA_REQUIRE(n_adapters > 0 && r_tot > 0, "residual_rmsnorm_shrink: bad adapter sizes");
  MLORA_REQUIRE(aligned16(d_res_in) && aligned16(d_res_out) && aligned16(d_w) && aligned16(d_out) && aligned16(d_A_all) &&
                    (!d_delta || aligned16(d_delta)),
                "residual_rmsnorm_shrink: pointers must be 16-byte aligned");
  if (T == 0) return MLORA_OK;
  MLORA_REQUIRE(T <= 65535, "residual_rmsnorm_shrink: T=%d exceeds 65535 rows per call", T);
  if (H <= 2 * kNsThreads * 8)
    launch_pdl_if(pdl_enabled_norm(), rmsnorm_shrink_kernel<2>, dim3(kNsSplit, T), dim3(kNsThreads), 0, (cudaStream_t)stream,
                  (const bf16*)d_delta, d_res_in, d_res_out, (const bf16*)d_w, eps, (bf16*)d_out, H, (const bf16*)d_A_all,
                  d_slots, n_adapters, r_tot, d_u);
  else
    launch_pdl_if(pdl_enabled_norm(), rmsnorm_shrink_kernel<4>, dim3(kNsSplit, T), dim3(kNsThreads), 0, (cudaStream_t)stream,
                  (const bf16*)d_delta, d_res_in, d_res_out, (const bf16*)d_w, eps, (bf16*)d_out, H, (const bf16*)d_A_all,
                  d_slots, n_adapters, r_tot, d_u);
  count_launch();
  MLORA_CHECK_LAUNCH("rmsnorm_shrink_kernel");
  return MLORA_OK;
}

extern "C" int mlora_embed(const int32_t* d_ids, const void* d_E, int32_t T, int32_t H, int32_t vocab,
                           float* d_res, void* d_out_bf16, void* stream) {
  MLORA_REQUIRE(T >= 0 && H > 0 && H % 8 == 0 && vocab > 0, "embed: bad sizes T=%d H=%d vocab=%d", T, H, vocab);
  MLORA_REQUIRE(d_ids && d_E && (d_res || d_out_bf16), "embed: null pointer");
  MLORA_REQUIRE(aligned16(d_E) && aligned16(d_res) && aligned16(d_out_bf16), "embed: pointers must be 16-byte aligned");
  if (T == 0) return MLORA_OK;
  launch_pdl(embed_kernel, T, 256, 0, (cudaStream_t)stream, d_ids, (const bf16*)d_E, H, vocab, d_res, (bf16*)d_out_bf16);
  count_launch();
  MLORA_CHECK_LAUNCH("embed_kernel");
  return MLORA_OK;
}

extern "C" int mlora_argmax(const float* d_logits, int64_t ld, int32_t T, int32_t V, int32_t* d_tok, void* stream) {
  MLORA_REQUIRE(T >= 0 && V > 0 && ld >= V, "argmax: bad sizes T=%d V=%d", T, V);
  MLORA_REQUIRE(d_logits && d_tok, "argmax: null pointer");
  if (T == 0) return MLORA_OK;
  launch_pdl(argmax_kernel, T, 1024, 0, (cudaStream_t)stream, d_logits, ld, V, d_tok);
  count_launch();
  MLORA_CHECK_LAUNCH("argmax_kernel");
  return MLORA_OK;
}

extern "C" int mlora_kv_begin_decode(const int32_t* d_row_slot, int32_t* d_seq_lens, int32_t* d_row_pos, int32_t B,
                                     void* stream) {
  MLORA_REQUIRE(B >= 0 && d_row_slot && d_seq_lens && d_row_pos, "kv_begin_decode: bad arguments");
  if (B == 0) return MLORA_OK;
  launch_pdl(kv_begin_decode_kernel, (B + 127) / 128, 128, 0, (cudaStream_t)stream, d_row_slot, d_seq_lens, d_row_pos, B);
  count_launch();
  MLORA_CHECK_LAUNCH("kv_begin_decode_kernel");
  return MLORA_OK;
}
