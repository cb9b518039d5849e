// Request -> adapter bucketing on the device: a stable counting sort of the rows of a batch by
// (has_adapter, adapter type, weight id), plus the compacted segment table the LoRA kernels and
// the decode-method selection need.  Integer work; results are bit-exact with a stable host sort.
//
// n <= 1024 rows (every decode step): one CTA, one launch, no scratch memory.
// larger n (prefill token batches): chunks of 1024 rows, three launches, per-chunk histograms in
// caller-provided scratch.
#include "common.cuh"

namespace mlora {
namespace {

constexpr int kChunk = 1024;
constexpr int kMaxKeys = 8192;  // shared-memory histogram bound

struct KeySpec {
  int n_types, n_wids, by_type, n_keys;
};

__device__ __forceinline__ int make_key(const int32_t* tids, const int32_t* wids, int i, const KeySpec& ks,
                                        int* tid_out, int* wid_out) {
  int wid = wids[i];
  int tid = tids ? tids[i] : (wid >= 0 ? 0 : -1);
  if (tid >= ks.n_types) tid = ks.n_types - 1;  // out-of-range ids are clamped, never dereferenced
  if (tid < 0) {
    *tid_out = -1;
    *wid_out = -1;
    return 0;
  }
  if (!ks.by_type) wid = min(max(wid, 0), ks.n_wids - 1);
  *tid_out = tid;
  *wid_out = wid;
  return ks.by_type ? 1 + tid : 1 + tid * ks.n_wids + wid;
}

// Exclusive scan of v[0..len) in shared memory by the whole CTA (blockDim.x threads, <= 1024).
// On return v holds the exclusive prefix and the total is returned to every thread.
__device__ int block_exclusive_scan(int* v, int len, int* warp_tot /*[33] smem*/) {
  const int tid = threadIdx.x, nt = blockDim.x;
  const int per = (len + nt - 1) / nt;
  const int b = min(tid * per, len), e = min(b + per, len);
  int s = 0;
  for (int i = b; i < e; ++i) s += v[i];
  // scan of per-thread sums
  int incl = s;
  const int lane = tid & 31, w = tid >> 5;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    int t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  if (lane == 31) warp_tot[w] = incl;
  __syncthreads();
  if (w == 0) {
    int t = (lane < (nt + 31) / 32) ? warp_tot[lane] : 0;
    int ti = t;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
      int u = __shfl_up_sync(0xffffffffu, ti, o);
      if (lane >= o) ti += u;
    }
    warp_tot[lane] = ti - t;  // exclusive per warp
    if (lane == 31) warp_tot[32] = ti;
  }
  __syncthreads();
  int run = warp_tot[w] + incl - s;
  for (int i = b; i < e; ++i) {
    int t = v[i];
    v[i] = run;
    run += t;
  }
  int total = warp_tot[32];
  __syncthreads();
  return total;
}

// Writes the segment table and the per-type counts from a scanned histogram.
//   base[k]  = first sorted position of key k (exclusive scan of the histogram), base[n_keys] = n
//   nz[k]    = number of non-empty keys before k (exclusive scan of hist>0)
__device__ void write_segments(const int* base, const int* nz, int n_seg, int n, const KeySpec& ks,
                               int32_t* seg_offsets, int32_t* seg_tid, int32_t* seg_wid, int32_t* counts) {
  for (int k = threadIdx.x; k < ks.n_keys; k += blockDim.x) {
    int cnt = base[k + 1] - base[k];
    if (cnt > 0) {
      int s = nz[k];
      seg_offsets[s] = base[k];
      int tid = -1, wid = -1;
      if (k > 0) {
        if (ks.by_type) {
          tid = k - 1;
          wid = -1;
        } else {
          tid = (k - 1) / ks.n_wids;
          wid = (k - 1) % ks.n_wids;
        }
      }
      seg_tid[s] = tid;
      seg_wid[s] = wid;
    }
  }
  if (threadIdx.x == 0) {
    seg_offsets[n_seg] = n;
    counts[0] = n_seg;
    counts[1] = base[1] - base[0];
  }
  for (int t = threadIdx.x; t < ks.n_types; t += blockDim.x) {
    int lo = ks.by_type ? 1 + t : 1 + t * ks.n_wids;
    int hi = ks.by_type ? 2 + t : 1 + (t + 1) * ks.n_wids;
    counts[2 + t] = base[hi] - base[lo];
  }
}

// ---- one-CTA path ------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) bucket_small_kernel(
    const int32_t* __restrict__ tids, const int32_t* __restrict__ wids, int n, KeySpec ks,
    int32_t* __restrict__ perm, int32_t* __restrict__ sorted_tid, int32_t* __restrict__ sorted_wid,
    int32_t* __restrict__ seg_offsets, int32_t* __restrict__ seg_tid, int32_t* __restrict__ seg_wid,
    int32_t* __restrict__ counts) {
  extern __shared__ int sm[];
  int* keys = sm;                    // [kChunk]
  int* base = keys + kChunk;         // [n_keys+1]
  int* nz = base + ks.n_keys + 1;    // [n_keys+1]
  __shared__ int warp_tot[33];
  const int i = threadIdx.x;
  for (int k = i; k <= ks.n_keys; k += blockDim.x) base[k] = 0;
  __syncthreads();
  int my_tid = -1, my_wid = -1, my_key = -1;
  if (i < n) {
    my_key = make_key(tids, wids, i, ks, &my_tid, &my_wid);
    keys[i] = my_key;
    atomicAdd(&base[my_key], 1);
  }
  __syncthreads();
  for (int k = i; k <= ks.n_keys; k += blockDim.x) nz[k] = (k < ks.n_keys && base[k] > 0) ? 1 : 0;
  __syncthreads();
  block_exclusive_scan(base, ks.n_keys + 1, warp_tot);  // base[n_keys] becomes n
  int n_seg = block_exclusive_scan(nz, ks.n_keys + 1, warp_tot);
  if (i < n) {
    int rank = 0;
    for (int j = 0; j < i; ++j) rank += (keys[j] == my_key);
    int pos = base[my_key] + rank;
    perm[pos] = i;
    if (sorted_tid) sorted_tid[pos] = my_tid;
    if (sorted_wid) sorted_wid[pos] = my_wid;
  }
  write_segments(base, nz, n_seg, n, ks, seg_offsets, seg_tid, seg_wid, counts);
}

// ---- chunked path --------------------------------------------------------------------------------
__global__ void __launch_bounds__(1024) bucket_hist_kernel(const int32_t* __restrict__ tids,
                                                           const int32_t* __restrict__ wids, int n,
                                                           KeySpec ks, int32_t* __restrict__ hist) {
  extern __shared__ int sm[];
  for (int k = threadIdx.x; k < ks.n_keys; k += blockDim.x) sm[k] = 0;
  __syncthreads();
  int i = blockIdx.x * kChunk + threadIdx.x;
  if (i < n) {
    int t, w;
    atomicAdd(&sm[make_key(tids, wids, i, ks, &t, &w)], 1);
  }
  __syncthreads();
  for (int k = threadIdx.x; k < ks.n_keys; k += blockDim.x) hist[(size_t)blockIdx.x * ks.n_keys + k] = sm[k];
}

// One CTA: turns per-chunk histograms into per-(chunk,key) start positions, in place.
__global__ void __launch_bounds__(1024) bucket_scan_kernel(int32_t* __restrict__ hist, int n_chunks, int n,
                                                           KeySpec ks, int32_t* __restrict__ seg_offsets,
                                                           int32_t* __restrict__ seg_tid,
                                                           int32_t* __restrict__ seg_wid,
                                                           int32_t* __restrict__ counts) {
  extern __shared__ int sm[];
  int* base = sm;                  // [n_keys+1]
  int* nz = base + ks.n_keys + 1;  // [n_keys+1]
  __shared__ int warp_tot[33];
  for (int k = threadIdx.x; k <= ks.n_keys; k += blockDim.x) {
    int tot = 0;
    if (k < ks.n_keys) {
      for (int c = 0; c < n_chunks; ++c) {
        int h = hist[(size_t)c * ks.n_keys + k];
        hist[(size_t)c * ks.n_keys + k] = tot;  // start of this chunk's rows inside key k
        tot += h;
      }
    }
    base[k] = tot;
    nz[k] = tot > 0 ? 1 : 0;
  }
  __syncthreads();
  block_exclusive_scan(base, ks.n_keys + 1, warp_tot);
  int n_seg = block_exclusive_scan(nz, ks.n_keys + 1, warp_tot);
  for (int k = threadIdx.x; k < ks.n_keys; k += blockDim.x)
    for (int c = 0; c < n_chunks; ++c) hist[(size_t)c * ks.n_keys + k] += base[k];
  write_segments(base, nz, n_seg, n, ks, seg_offsets, seg_tid, seg_wid, counts);
}

__global__ void __launch_bounds__(1024) bucket_scatter_kernel(
    const int32_t* __restrict__ tids, const int32_t* __restrict__ wids, int n, KeySpec ks,
    const int32_t* __restrict__ start, int32_t* __restrict__ perm, int32_t* __restrict__ sorted_tid,
    int32_t* __restrict__ sorted_wid) {
  __shared__ int keys[kChunk];
  int i = blockIdx.x * kChunk + threadIdx.x;
  int my_tid = -1, my_wid = -1, my_key = -1;
  if (i < n) {
    my_key = make_key(tids, wids, i, ks, &my_tid, &my_wid);
    keys[threadIdx.x] = my_key;
  }
  __syncthreads();
  if (i < n) {
    int rank = 0;
    for (int j = 0; j < (int)threadIdx.x; ++j) rank += (keys[j] == my_key);
    int pos = start[(size_t)blockIdx.x * ks.n_keys + my_key] + rank;
    perm[pos] = i;
    if (sorted_tid) sorted_tid[pos] = my_tid;
    if (sorted_wid) sorted_wid[pos] = my_wid;
  }
}

}  // namespace
}  // namespace mlora

using namespace mlora;

static int key_count(int n_types, int n_wids, int by_type) {
  return by_type ? n_types + 1 : 1 + n_types * n_wids;
}

extern "C" size_t mlora_bucket_sort_workspace(int32_t n, int32_t n_types, int32_t n_wids) {
  if (n <= kChunk) return 0;
  size_t chunks = ((size_t)n + kChunk - 1) / kChunk;
  return chunks * (size_t)key_count(n_types, n_wids, 0) * sizeof(int32_t);
}

extern "C" int mlora_bucket_sort(const int32_t* d_tids, const int32_t* d_wids, int32_t n, int32_t n_types,
                                 int32_t n_wids, int32_t by_type_only, int32_t* d_perm,
                                 int32_t* d_sorted_tid, int32_t* d_sorted_wid, int32_t* d_seg_offsets,
                                 int32_t* d_seg_tid, int32_t* d_seg_wid, int32_t* d_counts, void* d_work,
                                 size_t work_bytes, void* stream) {
  MLORA_REQUIRE(n >= 0 && n_types >= 0 && n_wids >= 1, "bucket_sort: bad sizes n=%d n_types=%d n_wids=%d", n,
                n_types, n_wids);
  MLORA_REQUIRE((n == 0 || (d_wids && d_perm)) && d_seg_offsets && d_seg_tid && d_seg_wid && d_counts,
                "bucket_sort: null pointer");
  if (!d_tids && n_types == 0) n_types = 1;
  KeySpec ks{n_types, n_wids, by_type_only ? 1 : 0, key_count(n_types, n_wids, by_type_only)};
  MLORA_REQUIRE(ks.n_keys <= kMaxKeys, "bucket_sort: %d keys exceed the limit of %d", ks.n_keys, kMaxKeys);
  cudaStream_t st = (cudaStream_t)stream;
  if (n <= kChunk) {
    size_t smem = (size_t)(kChunk + 2 * (ks.n_keys + 1)) * sizeof(int);
    if (smem > 48 * 1024)
      cudaFuncSetAttribute(bucket_small_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    bucket_small_kernel<<<1, 1024, smem, st>>>(d_tids, d_wids, n, ks, d_perm, d_sorted_tid, d_sorted_wid,
                                               d_seg_offsets, d_seg_tid, d_seg_wid, d_counts);
    count_launch();
    MLORA_CHECK_LAUNCH("bucket_small_kernel");
    return MLORA_OK;
  }
  int chunks = (n + kChunk - 1) / kChunk;
  size_t need = (size_t)chunks * ks.n_keys * sizeof(int32_t);
  if (!d_work || work_bytes < need)
    return fail(MLORA_ESIZE, "bucket_sort: workspace of %zu bytes needed, %zu given", need, work_bytes);
  int32_t* hist = (int32_t*)d_work;
  bucket_hist_kernel<<<chunks, 1024, ks.n_keys * sizeof(int), st>>>(d_tids, d_wids, n, ks, hist);
  size_t smem = (size_t)(2 * (ks.n_keys + 1)) * sizeof(int);
  if (smem > 48 * 1024)
    cudaFuncSetAttribute(bucket_scan_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
  bucket_scan_kernel<<<1, 1024, smem, st>>>(hist, chunks, n, ks, d_seg_offsets, d_seg_tid, d_seg_wid,
                                            d_counts);
  bucket_scatter_kernel<<<chunks, 1024, 0, st>>>(d_tids, d_wids, n, ks, hist, d_perm, d_sorted_tid,
                                                 d_sorted_wid);
  count_launch(3);
  MLORA_CHECK_LAUNCH("bucket_sort (chunked)");
  return MLORA_OK;
}
