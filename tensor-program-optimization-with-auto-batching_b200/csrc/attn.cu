// Paged-KV attention for single-query rows (decode, and prefill rows after their K/V were
// appended), RoPE + KV append, and the split-KV merge.
//
// Cache layout per layer: K pages [n_pages, Hkv, page_size, D] bf16, V pages alike, so one
// (page, head) holds page_size*D contiguous elements (4 KB at page 16, D 128).  A warp streams a
// page with 128-bit loads: D/8 lanes cover one token, 32/(D/8) tokens per load instruction; all K
// and V loads of a page are issued before the first use.  Scores are reduced inside each lane
// group with xor-shuffles; every lane group keeps its own online-softmax state (m, l, acc[8]);
// groups, warps and splits are merged at the end.
#include <cmath>
#include <mutex>

#include "common.cuh"

namespace mlora {
namespace {

constexpr float kLog2e = 1.4426950408889634f;

struct AttnArgs {
  const bf16* qkv;
  int64_t ld;
  bf16* k_pages;
  bf16* v_pages;
  const int32_t* block_table;
  int max_pages;
  const int32_t* row_slot;
  const int32_t* row_pos;
  int T, Hq, Hkv, page_size;
  float theta;
  int fused;
  bf16* out;
  int64_t ld_out;
  int n_splits;
  float* work;
  // optional: the LoRA shrink of the projection that reads `out` (o_proj), computed in this kernel's tail
  const bf16* sh_A;            // [N, sh_r, Hq*D] or nullptr
  const int32_t* sh_slots;     // [T]
  int sh_n_adapters, sh_r;
  float* sh_u;                 // [T, sh_r]
  float* sh_part;              // [T, Hq, sh_r] per-head partial dot products
  int32_t* sh_tickets;         // [T], zero between calls
};

// K/V pages are read once per step: no L1 allocation, and first in line for L2 eviction (`pol`), so that gigabytes
// of pages per step do not push the activations and the next kernel's instructions out of L2.
__device__ __forceinline__ uint64_t kv_policy() {
  uint64_t pol;
  asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
  return pol;
}
__device__ __forceinline__ uint4 ld_kv(const void* p, uint64_t pol) {
  uint4 v;
  asm volatile("ld.global.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(p), "l"(pol));
  return v;
}

__device__ __forceinline__ float rope_inv_freq(float theta, int i, int D) {
  // theta^(-2i/D), evaluated in fp32 like the reference frameworks do
  return powf(theta, -(float)(2 * i) / (float)D);
}

__device__ __forceinline__ void merge_state(float& m, float& l, float (&acc)[8], float mo, float lo,
                                            const float (&acco)[8]) {
  const float mn = fmaxf(m, mo);
  const float c1 = (m == -INFINITY) ? 0.f : exp2f(m - mn);
  const float c2 = (mo == -INFINITY) ? 0.f : exp2f(mo - mn);
  l = l * c1 + lo * c2;
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = acc[e] * c1 + acco[e] * c2;
  m = mn;
}

// grid (Hq, T, n_splits), 128 threads.  IT = page_size / tokens-per-load.
template <int D, int IT>
__global__ void __launch_bounds__(128) paged_attn_kernel(AttnArgs a) {
  constexpr int LPT = D / 8;    // lanes per token
  constexpr int TPW = 32 / LPT; // tokens per warp-wide load
  constexpr int PS = IT * TPW;  // page size
  __shared__ float sq[D];       // rotated, scaled query
  __shared__ float sk[D];       // rotated new key (bf16-rounded)
  __shared__ float sv[D];       // new value
  __shared__ float wm[4], wl[4];
  __shared__ float wacc[4][D];
  __shared__ float s_new;

  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, t = blockIdx.y, split = blockIdx.z;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int rep = a.Hq / a.Hkv, kvh = h / rep;
  const int slot = a.row_slot[t], pos = a.row_pos[t];
  const int32_t* bt = a.block_table + (size_t)slot * a.max_pages;
  const bf16* row = a.qkv + (size_t)t * a.ld;
  const float qscale = rsqrtf((float)D) * kLog2e;
  const bool last_split = split == a.n_splits - 1;
  const bool has_new = a.fused && last_split;
  // A position beyond the row's block-table entries (a step issued without reserved pages) is never
  // dereferenced: the new k/v are not stored and the context is cut at the table's end.
  const bool can_store = pos >= 0 && pos / PS < a.max_pages;

  // ---- prologue: rotate q (and the new k), stage the new k/v -----------------------------------
  if (tid < D / 2) {
    const int i = tid;
    float q1 = __bfloat162float(row[h * D + i]), q2 = __bfloat162float(row[h * D + i + D / 2]);
    if (a.fused) {
      float sn, cs;
      sincosf((float)pos * rope_inv_freq(a.theta, i, D), &sn, &cs);
      const float r1 = q1 * cs - q2 * sn, r2 = q2 * cs + q1 * sn;
      q1 = r1, q2 = r2;
    }
    sq[i] = q1 * qscale;
    sq[i + D / 2] = q2 * qscale;
  } else if (tid < D && has_new) {
    const int i = tid - D / 2;
    const bf16* kr = row + (size_t)(a.Hq + kvh) * D;
    const float k1 = __bfloat162float(kr[i]), k2 = __bfloat162float(kr[i + D / 2]);
    float sn, cs;
    sincosf((float)pos * rope_inv_freq(a.theta, i, D), &sn, &cs);
    const bf16 r1 = __float2bfloat16_rn(k1 * cs - k2 * sn), r2 = __float2bfloat16_rn(k2 * cs + k1 * sn);
    sk[i] = __bfloat162float(r1);
    sk[i + D / 2] = __bfloat162float(r2);
    if (h % rep == 0 && can_store) {
      const int page = bt[pos / PS];
      bf16* dst = a.k_pages + (((size_t)page * a.Hkv + kvh) * PS + pos % PS) * D;
      dst[i] = r1;
      dst[i + D / 2] = r2;
    }
  }
  if (has_new && tid < D) {
    const bf16 v = row[(size_t)(a.Hq + a.Hkv + kvh) * D + tid];
    sv[tid] = __bfloat162float(v);
    if (h % rep == 0 && can_store) {
      const int page = bt[pos / PS];
      a.v_pages[(((size_t)page * a.Hkv + kvh) * PS + pos % PS) * D + tid] = v;
    }
  }
  __syncthreads();

  const int g = lane / LPT, dl = lane % LPT;
  float qf[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) qf[e] = sq[dl * 8 + e];

  // tokens read from the pages: [0, n_tok)
  const int n_tok = min(max(a.fused ? pos : pos + 1, 0), a.max_pages * PS);
  const int n_pg = (n_tok + PS - 1) / PS;
  const int per = (n_pg + a.n_splits - 1) / a.n_splits;
  const int pg_begin = min(split * per, n_pg), pg_end = min(pg_begin + per, n_pg);

  float m = -INFINITY, l = 0.f, acc[8];
#pragma unroll
  for (int e = 0; e < 8; ++e) acc[e] = 0.f;

  const uint64_t pol = kv_policy();
  for (int pg = pg_begin + warp; pg < pg_end; pg += 4) {
    const int page = bt[pg];
    const size_t base = ((size_t)page * a.Hkv + kvh) * PS * D + (size_t)g * D + dl * 8;
    const bf16* kp = a.k_pages + base;
    const bf16* vp = a.v_pages + base;
    uint4 kr[IT], vr[IT];
#pragma unroll
    for (int it = 0; it < IT; ++it) kr[it] = ld_kv(kp + (size_t)it * TPW * D, pol);
#pragma unroll
    for (int it = 0; it < IT; ++it) vr[it] = ld_kv(vp + (size_t)it * TPW * D, pol);
    float s[IT];
    float mx = -INFINITY;
#pragma unroll
    for (int it = 0; it < IT; ++it) {
      float kf[8];
      unpack8(kr[it], kf);
      float d = 0.f;
#pragma unroll
      for (int e = 0; e < 8; ++e) d = fmaf(qf[e], kf[e], d);
#pragma unroll
      for (int o = LPT / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
      const bool valid = pg * PS + it * TPW + g < n_tok;
      s[it] = valid ? d : -INFINITY;
      mx = fmaxf(mx, s[it]);
    }
    const float mn = fmaxf(m, mx);
    if (mn != -INFINITY) {
      const float corr = (m == -INFINITY) ? 0.f : exp2f(m - mn);
      l *= corr;
#pragma unroll
      for (int e = 0; e < 8; ++e) acc[e] *= corr;
#pragma unroll
      for (int it = 0; it < IT; ++it) {
        if (s[it] != -INFINITY) {
          const float p = exp2f(s[it] - mn);
          float vf[8];
          unpack8(vr[it], vf);
          l += p;
#pragma unroll
          for (int e = 0; e < 8; ++e) acc[e] = fmaf(p, vf[e], acc[e]);
        }
      }
      m = mn;
    }
  }

  // ---- merge the lane groups of the warp -------------------------------------------------------
#pragma unroll
  for (int o = LPT; o < 32; o <<= 1) {
    const float mo = __shfl_xor_sync(0xffffffffu, m, o);
    const float lo = __shfl_xor_sync(0xffffffffu, l, o);
    float ao[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) ao[e] = __shfl_xor_sync(0xffffffffu, acc[e], o);
    merge_state(m, l, acc, mo, lo, ao);
  }
  if (lane < LPT) {
    if (lane == 0) {
      wm[warp] = m;
      wl[warp] = l;
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) wacc[warp][lane * 8 + e] = acc[e];
  }
  if (warp == 0 && has_new) {
    float d = 0.f;
    for (int i = lane; i < D; i += 32) d = fmaf(sq[i], sk[i], d);
    d = warp_sum(d);
    if (lane == 0) s_new = d;
  }
  __syncthreads();

  // ---- merge warps (+ the new token) and write -------------------------------------------------
  float o_val = 0.f;
  if (tid < D) {
    float M = has_new ? s_new : -INFINITY;
#pragma unroll
    for (int w = 0; w < 4; ++w) M = fmaxf(M, wm[w]);
    float L = 0.f, O = 0.f;
    if (M != -INFINITY) {
#pragma unroll
      for (int w = 0; w < 4; ++w) {
        const float c = (wm[w] == -INFINITY) ? 0.f : exp2f(wm[w] - M);
        L = fmaf(wl[w], c, L);
        O = fmaf(wacc[w][tid], c, O);
      }
      if (has_new) {
        const float c = exp2f(s_new - M);
        L += c;
        O = fmaf(sv[tid], c, O);
      }
    }
    if (a.n_splits == 1) {
      const bf16 ob = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
      a.out[(size_t)t * a.ld_out + h * D + tid] = ob;
      o_val = __bfloat162float(ob);  // exactly what a separate shrink kernel would read back
    } else {
      float* w = a.work + (((size_t)t * a.Hq + h) * a.n_splits + split) * (D + 2);
      w[tid] = O;
      if (tid == 0) {
        w[D] = M;
        w[D + 1] = L;
      }
    }
  }
  // ---- optional tail: u[t, j] = A[slot, j, :] . out[t, :] for the projection that reads this output ------------------
  // Every (row, head) CTA multiplies its 128 outputs with the matching columns of the adapter's A rows (they are
  // L2 resident: the K/V stream is marked evict-first) and leaves per-head partial sums; the last head of a row to
  // arrive adds them up in head order.  One launch less per layer than a separate shrink kernel, and none of its
  // round trips on the critical path between attention and projection.
  if (a.sh_A != nullptr && a.n_splits == 1) {
    __shared__ int s_last;
    const int r = a.sh_r;
    const int slot = a.sh_slots[t];
    const bool has = slot >= 0 && slot < a.sh_n_adapters;
    float* part = a.sh_part + ((size_t)t * a.Hq + h) * r;
    __syncthreads();  // wacc is reused below
    float* sred = &wacc[0][0];  // [4][16]
    for (int j0 = 0; j0 < r; j0 += 16) {
      if (has) {
        const bf16* arow = a.sh_A + ((size_t)slot * r + j0) * ((size_t)a.Hq * D) + (size_t)h * D + tid;
        float p[16];
#pragma unroll
        for (int jj = 0; jj < 16; ++jj)
          p[jj] = (tid < D && j0 + jj < r) ? o_val * __bfloat162float(arow[(size_t)jj * a.Hq * D]) : 0.f;
#pragma unroll
        for (int jj = 0; jj < 16; ++jj) p[jj] = warp_sum(p[jj]);
        if (lane == 0) {
#pragma unroll
          for (int jj = 0; jj < 16; ++jj) sred[warp * 16 + jj] = p[jj];
        }
      }
      __syncthreads();
      if (tid < 16 && j0 + tid < r)
        part[j0 + tid] = has ? (sred[tid] + sred[16 + tid]) + (sred[32 + tid] + sred[48 + tid]) : 0.f;
      __syncthreads();
    }
    __threadfence();
    __syncthreads();
    if (tid == 0) {
      const int old = atomicAdd(&a.sh_tickets[t], 1);
      s_last = old == a.Hq - 1;
      if (s_last) a.sh_tickets[t] = 0;  // ready for the next call
    }
    __syncthreads();
    if (s_last) {
      __threadfence();
      for (int j = tid; j < r; j += blockDim.x) {
        float acc = 0.f;
        for (int hh = 0; hh < a.Hq; ++hh) acc += __ldcg(a.sh_part + ((size_t)t * a.Hq + hh) * r + j);  // head order
        a.sh_u[(size_t)t * r + j] = acc;
      }
    }
  }
}

// grid (Hq, T), D threads: combine the n_splits partial results of one (row, head).
__global__ void attn_merge_kernel(const float* __restrict__ work, int Hq, int D, int n_splits,
                                  bf16* __restrict__ out, int64_t ld_out) {
  pdl_launch_dependents();
  pdl_wait();
  const int h = blockIdx.x, t = blockIdx.y, d = threadIdx.x;
  const float* w = work + ((size_t)t * Hq + h) * n_splits * (D + 2);
  float M = -INFINITY;
  for (int s = 0; s < n_splits; ++s) M = fmaxf(M, w[(size_t)s * (D + 2) + D]);
  float L = 0.f, O = 0.f;
  if (M != -INFINITY) {
    for (int s = 0; s < n_splits; ++s) {
      const float ms = w[(size_t)s * (D + 2) + D];
      const float c = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
      L = fmaf(w[(size_t)s * (D + 2) + D + 1], c, L);
      O = fmaf(w[(size_t)s * (D + 2) + d], c, O);
    }
  }
  out[(size_t)t * ld_out + h * D + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
}

// grid (T), 256 threads: rotate q in place, rotate k into the pages, copy v into the pages.
__global__ void __launch_bounds__(256) kv_append_rope_kernel(bf16* __restrict__ qkv, int64_t ld,
                                                             bf16* __restrict__ k_pages, bf16* __restrict__ v_pages,
                                                             const int32_t* __restrict__ block_table, int max_pages,
                                                             const int32_t* __restrict__ row_slot,
                                                             const int32_t* __restrict__ row_pos, int Hq, int Hkv,
                                                             int D, int PS, float theta) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const int slot = row_slot[t], pos = row_pos[t];
  if (pos < 0 || pos / PS >= max_pages) return;  // no block-table entry for this position: nothing is written
  const int page = block_table[(size_t)slot * max_pages + pos / PS];
  bf16* row = qkv + (size_t)t * ld;
  const int half = D / 2;
  // a thread keeps one pair of adjacent frequencies (its sine / cosine computed once) and walks the heads
  const int pairs = half / 2;                       // 4-byte column pairs per half head
  const int i = (threadIdx.x % pairs) * 2;
  float sn0, cs0, sn1, cs1;
  sincosf((float)pos * rope_inv_freq(theta, i, D), &sn0, &cs0);
  sincosf((float)pos * rope_inv_freq(theta, i + 1, D), &sn1, &cs1);
  for (int head = threadIdx.x / pairs; head < Hq + Hkv; head += blockDim.x / pairs) {
    bf16* p = row + (size_t)head * D;
    const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(p + i);
    const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(p + i + half);
    const float x1a = __bfloat162float(a.x), x1b = __bfloat162float(a.y);
    const float x2a = __bfloat162float(b.x), x2b = __bfloat162float(b.y);
    __nv_bfloat162 r1, r2;
    r1.x = __float2bfloat16_rn(x1a * cs0 - x2a * sn0);
    r1.y = __float2bfloat16_rn(x1b * cs1 - x2b * sn1);
    r2.x = __float2bfloat16_rn(x2a * cs0 + x1a * sn0);
    r2.y = __float2bfloat16_rn(x2b * cs1 + x1b * sn1);
    bf16* dst = head < Hq ? p : k_pages + (((size_t)page * Hkv + (head - Hq)) * PS + pos % PS) * D;
    *reinterpret_cast<__nv_bfloat162*>(dst + i) = r1;
    *reinterpret_cast<__nv_bfloat162*>(dst + i + half) = r2;
  }
  const bf16* vsrc = row + (size_t)(Hq + Hkv) * D;
  for (int idx = threadIdx.x; idx < Hkv * D / 8; idx += blockDim.x) {
    const int head = (idx * 8) / D, d = (idx * 8) % D;
    bf16* dst = v_pages + (((size_t)page * Hkv + head) * PS + pos % PS) * D + d;
    *reinterpret_cast<uint4*>(dst) = *reinterpret_cast<const uint4*>(vsrc + (size_t)head * D + d);
  }
}

int pick_splits(int T, int Hq, int max_pages) {
  const int base = T * Hq;
  if (base >= 592) return 1;  // >= 4 CTAs on each of the 148 SMs already
  int s = (592 + base - 1) / base;
  s = s > 16 ? 16 : s;
  const int by_ctx = max_pages / 4 > 0 ? max_pages / 4 : 1;
  return s < by_ctx ? s : by_ctx;
}

}  // namespace
}  // namespace mlora

using namespace mlora;

extern "C" size_t mlora_paged_attention_workspace(int32_t T, int32_t Hq, int32_t D, int32_t n_splits) {
  if (n_splits <= 0) n_splits = 16;
  if (n_splits == 1) return 0;
  return (size_t)T * Hq * n_splits * (D + 2) * sizeof(float);
}

static int check_kv_common(const char* who, int T, int Hq, int Hkv, int D, int page_size) {
  MLORA_REQUIRE(T >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0, "%s: bad head counts Hq=%d Hkv=%d", who, Hq, Hkv);
  MLORA_REQUIRE(D == 64 || D == 128, "%s: head_dim %d not supported (64 or 128)", who, D);
  MLORA_REQUIRE(page_size == 16 || page_size == 32, "%s: page_size %d not supported (16 or 32)", who, page_size);
  return MLORA_OK;
}

extern "C" int mlora_kv_append_rope(void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                    const int32_t* d_block_table, int32_t max_pages, const int32_t* d_row_slot,
                                    const int32_t* d_row_pos, int32_t T, int32_t Hq, int32_t Hkv, int32_t D,
                                    int32_t page_size, float rope_theta, void* stream) {
  int rc = check_kv_common("kv_append_rope", T, Hq, Hkv, D, page_size);
  if (rc) return rc;
  MLORA_REQUIRE(d_qkv && d_k_pages && d_v_pages && d_block_table && d_row_slot && d_row_pos && max_pages > 0,
                "kv_append_rope: null pointer");
  MLORA_REQUIRE(ld % 8 == 0 && aligned16(d_qkv) && aligned16(d_v_pages), "kv_append_rope: alignment");
  if (T == 0) return MLORA_OK;
  launch_pdl(kv_append_rope_kernel, T, 256, 0, (cudaStream_t)stream, (bf16*)d_qkv, ld, (bf16*)d_k_pages, (bf16*)d_v_pages,
                                                             d_block_table, max_pages, d_row_slot, d_row_pos, Hq, Hkv,
                                                             D, page_size, rope_theta);
  count_launch();
  MLORA_CHECK_LAUNCH("kv_append_rope_kernel");
  return MLORA_OK;
}

struct ShrinkTail {
  const void* A = nullptr;
  const int32_t* slots = nullptr;
  int n_adapters = 0, r = 0;
  float* u = nullptr;
  float* part = nullptr;
  int32_t* tickets = nullptr;
};

static int attention_impl(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                          const int32_t* d_block_table, int32_t max_pages, const int32_t* d_row_slot,
                          const int32_t* d_row_pos, int32_t T, int32_t Hq, int32_t Hkv, int32_t D,
                          int32_t page_size, float rope_theta, int32_t fused_append, void* d_out,
                          int64_t ld_out, int32_t n_splits, void* d_work, size_t work_bytes,
                          void* stream, const ShrinkTail& sh) {
  int rc = check_kv_common("paged_attention", T, Hq, Hkv, D, page_size);
  if (rc) return rc;
  MLORA_REQUIRE(d_qkv && d_k_pages && d_v_pages && d_block_table && d_row_slot && d_row_pos && d_out && max_pages > 0,
                "paged_attention: null pointer");
  MLORA_REQUIRE(aligned16(d_k_pages) && aligned16(d_v_pages), "paged_attention: pages must be 16-byte aligned");
  if (T == 0) return MLORA_OK;
  MLORA_REQUIRE(T <= 65535, "paged_attention: T=%d exceeds 65535 rows per call", T);
  if (n_splits <= 0) {
    n_splits = pick_splits(T, Hq, max_pages);
    while (n_splits > 1 && mlora_paged_attention_workspace(T, Hq, D, n_splits) > work_bytes) --n_splits;
  }
  MLORA_REQUIRE(n_splits <= 64, "paged_attention: n_splits=%d exceeds 64", n_splits);
  if (n_splits > 1) {
    size_t need = mlora_paged_attention_workspace(T, Hq, D, n_splits);
    if (!d_work || work_bytes < need)
      return fail(MLORA_ESIZE, "paged_attention: workspace of %zu bytes needed, %zu given", need, work_bytes);
  }
  AttnArgs a{(const bf16*)d_qkv, ld, (bf16*)d_k_pages, (bf16*)d_v_pages, d_block_table, max_pages, d_row_slot,
             d_row_pos, T, Hq, Hkv, page_size, rope_theta, fused_append ? 1 : 0, (bf16*)d_out, ld_out, n_splits,
             (float*)d_work, (const bf16*)sh.A, sh.slots, sh.n_adapters, sh.r, sh.u, sh.part, sh.tickets};
  dim3 grid(Hq, T, n_splits);
  cudaStream_t st = (cudaStream_t)stream;
  if (D == 128 && page_size == 16)
    launch_pdl_if(pdl_enabled_attn(), paged_attn_kernel<128, 8>, grid, 128, 0, st, a);
  else if (D == 128 && page_size == 32)
    launch_pdl_if(pdl_enabled_attn(), paged_attn_kernel<128, 16>, grid, 128, 0, st, a);
  else if (D == 64 && page_size == 16)
    launch_pdl_if(pdl_enabled_attn(), paged_attn_kernel<64, 4>, grid, 128, 0, st, a);
  else
    launch_pdl_if(pdl_enabled_attn(), paged_attn_kernel<64, 8>, grid, 128, 0, st, a);
  count_launch();
  if (n_splits > 1) {
    launch_pdl_if(pdl_enabled_attn(), attn_merge_kernel, dim3(Hq, T), D, 0, st, (const float*)d_work, Hq, D, n_splits, (bf16*)d_out, ld_out);
    count_launch();
  }
  MLORA_CHECK_LAUNCH("paged_attn_kernel");
  return MLORA_OK;
}

extern "C" int mlora_paged_attention(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                     const int32_t* d_block_table, int32_t max_pages, const int32_t* d_row_slot,
                                     const int32_t* d_row_pos, int32_t T, int32_t Hq, int32_t Hkv, int32_t D,
                                     int32_t page_size, float rope_theta, int32_t fused_append, void* d_out,
                                     int64_t ld_out, int32_t n_splits, void* d_work, size_t work_bytes,
                                     void* stream) {
  return attention_impl(d_qkv, ld, d_k_pages, d_v_pages, d_block_table, max_pages, d_row_slot, d_row_pos, T, Hq, Hkv, D,
                        page_size, rope_theta, fused_append, d_out, ld_out, n_splits, d_work, work_bytes, stream,
                        ShrinkTail{});
}

extern "C" uint32_t mlora_paged_attention_splits(int32_t T, int32_t Hq, int32_t max_pages) {
  if (T <= 0 || Hq <= 0 || max_pages <= 0) return 1;
  return (uint32_t)pick_splits(T, Hq, max_pages);
}

extern "C" size_t mlora_paged_attention_shrink_workspace(int32_t T, int32_t Hq, int32_t r_max) {
  if (T <= 0 || Hq <= 0 || r_max <= 0) return 0;
  return (((size_t)T * sizeof(int32_t) + 255) & ~(size_t)255) + (size_t)T * Hq * r_max * sizeof(float);
}

extern "C" int mlora_paged_attention_shrink(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                            const int32_t* d_block_table, int32_t max_pages,
                                            const int32_t* d_row_slot, const int32_t* d_row_pos, int32_t T, int32_t Hq,
                                            int32_t Hkv, int32_t D, int32_t page_size, float rope_theta,
                                            int32_t fused_append, void* d_out, int64_t ld_out, const void* d_A_all,
                                            const int32_t* d_ranks, const int32_t* d_slots, int32_t n_adapters,
                                            int32_t r_max, float* d_u, void* d_shrink_work, size_t shrink_work_bytes,
                                            void* stream) {
  MLORA_REQUIRE(d_A_all && d_ranks && d_slots && d_u && d_shrink_work && n_adapters > 0 && r_max > 0 && r_max % 8 == 0,
                "paged_attention_shrink: LoRA operands");
  MLORA_REQUIRE(T >= 0 && Hq > 0, "paged_attention_shrink: bad sizes");
  const size_t need = mlora_paged_attention_shrink_workspace(T, Hq, r_max);
  if (shrink_work_bytes < need)
    return fail(MLORA_ESIZE, "paged_attention_shrink: workspace of %zu bytes needed, %zu given", need, shrink_work_bytes);
  if (T > 0 && pick_splits(T, Hq, max_pages) != 1) {
    // few rows: the attention is split over the context and merged by a second kernel; the shrink then runs as its own
    MLORA_REQUIRE(false, "paged_attention_shrink: %d rows x %d heads leave SMs idle, the split-context form is needed: "
                         "call mlora_paged_attention and mlora_lora_shrink", T, Hq);
  }
  ShrinkTail sh;
  sh.A = d_A_all;
  sh.slots = d_slots;
  sh.n_adapters = n_adapters;
  sh.r = r_max;
  sh.u = d_u;
  sh.tickets = (int32_t*)d_shrink_work;
  sh.part = (float*)((uint8_t*)d_shrink_work + (((size_t)T * sizeof(int32_t) + 255) & ~(size_t)255));
  return attention_impl(d_qkv, ld, d_k_pages, d_v_pages, d_block_table, max_pages, d_row_slot, d_row_pos, T, Hq, Hkv, D,
                        page_size, rope_theta, fused_append, d_out, ld_out, 1, nullptr, 0, stream, sh);
}

// ---- allocation-free variant -------------------------------------------------------------------------
// Scratch for the split-KV partial results lives in the library image itself, so a caller that is not
// allowed to allocate device memory can still use the split-KV path.  Every GPU that loads the library
// carries this array until the process exits.
namespace {
constexpr size_t kStaticScratchBytes = (size_t)16 << 20;  // 16 MiB
static __device__ __align__(256) unsigned char g_attn_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_static_mu;
void* g_static_ptr[kMaxDevices] = {};
bool g_static_ready[kMaxDevices] = {};

// Device address of the array on the current device.  In host code the array's name is only a handle,
// not an address a kernel could use; the runtime has to translate it, once per device, with that
// device current.
int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return fail(MLORA_ECUDA, "paged_attention_static: cudaGetDevice: %s", cudaGetErrorString(e));
  if (dev < 0 || dev >= kMaxDevices)
    return fail(MLORA_EINVAL, "paged_attention_static: device ordinal %d not supported (limit %d)", dev, kMaxDevices);
  std::lock_guard<std::mutex> lock(g_static_mu);
  if (!g_static_ready[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_attn_static_scratch);
    if (e != cudaSuccess || p == nullptr)
      return fail(MLORA_ECUDA, "paged_attention_static: cudaGetSymbolAddress: %s", cudaGetErrorString(e));
    g_static_ptr[dev] = p;
    g_static_ready[dev] = true;
  }
  *out = g_static_ptr[dev];
  return MLORA_OK;
}
}  // namespace

extern "C" size_t mlora_paged_attention_static_max_bytes(void) { return kStaticScratchBytes; }

extern "C" int mlora_paged_attention_static(const void* d_qkv, int64_t ld, void* d_k_pages, void* d_v_pages,
                                            const int32_t* d_block_table, int32_t max_pages,
                                            const int32_t* d_row_slot, const int32_t* d_row_pos, int32_t T,
                                            int32_t Hq, int32_t Hkv, int32_t D, int32_t page_size, float rope_theta,
                                            int32_t fused_append, void* d_out, int64_t ld_out, int32_t n_splits,
                                            void* stream) {
  // argument checks first (a negative size must come back as an invalid argument, not as a size problem)
  int rc = check_kv_common("paged_attention_static", T, Hq, Hkv, D, page_size);
  if (rc) return rc;
  MLORA_REQUIRE(T <= 65535, "paged_attention_static: T=%d exceeds 65535 rows per call", T);
  MLORA_REQUIRE(n_splits <= 64, "paged_attention_static: n_splits=%d exceeds 64", n_splits);
  if (n_splits > 1) {
    const size_t need = mlora_paged_attention_workspace(T, Hq, D, n_splits);
    if (need > kStaticScratchBytes)
      return fail(MLORA_ESIZE,
                  "paged_attention_static: %d rows x %d heads x %d splits need %zu bytes of scratch, the built-in "
                  "array holds %zu; use fewer splits or rows, or mlora_paged_attention with your own buffer",
                  T, Hq, n_splits, need, kStaticScratchBytes);
  }
  void* scratch = nullptr;
  rc = static_scratch_for_current_device(&scratch);
  if (rc) return rc;
  // n_splits <= 0: the library picks the split count and lowers it until the partials fit the array
  return mlora_paged_attention(d_qkv, ld, d_k_pages, d_v_pages, d_block_table, max_pages, d_row_slot, d_row_pos, T, Hq,
                               Hkv, D, page_size, rope_theta, fused_append, d_out, ld_out, n_splits, scratch,
                               kStaticScratchBytes, stream);
}
