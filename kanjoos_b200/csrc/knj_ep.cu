// knj_ep.cu -- kernels around the expert-parallel exchange. Two exchanges are served.
// "dispatch": rows are packed in (destination rank, expert, pair) order before a per-pair all-to-all, and the
// receiving rank turns the per-source expert counts into its local grouped-GEMM plan.
// "gather": every rank holds all token rows (all-gather), computes its experts' pairs, forms per-token partial
// sums over its experts (ep_combine_partial) and the ranks' partial rows are summed in rank order (ep_reduce). The reference has no multi-GPU path (it keeps every expert on one
// device: docs/01-architecture.md:322-325); these entry points serve the
// expert-sharded layout this library adds, and follow the pair/plan conventions
// of the single-device path (tools/bench/q4k_stream_ffn.hip:957-1001).
#include "knj_common.cuh"

using namespace knj;

namespace {

// send_off[e] = number of pairs routed to experts < e (exclusive scan of
// pair_cnt), one CTA. E <= 256.
__global__ void __launch_bounds__(256) ep_offsets_kernel(const int32_t *__restrict__ pair_cnt, int E,
                                                         int32_t *__restrict__ send_off) {
  __shared__ int s[256];
  const int e = threadIdx.x;
  s[e] = e < E ? pair_cnt[e] : 0;
  __syncthreads();
  if (e == 0) {
    int run = 0;
    for (int i = 0; i < E; ++i) { const int c = s[i]; s[i] = run; run += c; }
    send_off[E] = run;
  }
  __syncthreads();
  if (e < E) send_off[e] = s[e];
}

// One CTA per send slot group: copies the hidden row of every pair into the
// send buffer in expert-major order and records where each pair went.
__global__ void __launch_bounds__(256) ep_pack_kernel(const uint4 *__restrict__ x, int64_t row_u4, int top_k,
                                                      const int32_t *__restrict__ pair_idx, int idx_stride,
                                                      const int32_t *__restrict__ pair_cnt,
                                                      const int32_t *__restrict__ send_off, int E,
                                                      uint4 *__restrict__ send_rows, int32_t *__restrict__ pair_row) {
  const int e = blockIdx.y;
  const int cnt = pair_cnt[e];
  const int base = send_off[e];
  for (int i = blockIdx.x; i < cnt; i += gridDim.x) {
    const int p = pair_idx[(size_t)e * idx_stride + i];
    const uint4 *src = x + (size_t)(p / top_k) * row_u4;
    uint4 *dst = send_rows + (size_t)(base + i) * row_u4;
    for (int j = threadIdx.x; j < row_u4; j += 256) dst[j] = __ldg(src + j);
    if (threadIdx.x == 0) pair_row[p] = base + i;
  }
}

// Local plan of the receiving rank. counts[r][e] = rows rank r sends for my
// local expert e; rows from rank r arrive contiguously, experts ascending. One
// CTA per local expert lists its rows (source ranks in ascending order).
__global__ void __launch_bounds__(256) ep_plan_kernel(const int32_t *__restrict__ counts, int G, int E_loc,
                                                      int idx_stride, int32_t *__restrict__ pair_idx,
                                                      int32_t *__restrict__ pair_cnt) {
  const int e = blockIdx.x;
  __shared__ int src_base[64];  // first received row of (rank r, expert e)
  __shared__ int dst_base[65];
  if (threadIdx.x == 0) {
    int row = 0, mine = 0;
    for (int r = 0; r < G; ++r) {
      int before = 0, all = 0;
      for (int j = 0; j < E_loc; ++j) {
        const int c = counts[r * E_loc + j];
        if (j < e) before += c;
        all += c;
      }
      src_base[r] = row + before;
      dst_base[r] = mine;
      mine += counts[r * E_loc + e];
      row += all;
    }
    dst_base[G] = mine;
  }
  __syncthreads();
  int32_t *out = pair_idx + (size_t)e * idx_stride;
  const int total = min(dst_base[G], idx_stride);
  for (int r = 0; r < G; ++r) {
    const int c = dst_base[r + 1] - dst_base[r];
    for (int i = threadIdx.x; i < c; i += 256)
      if (dst_base[r] + i < idx_stride) out[dst_base[r] + i] = src_base[r] + i;
  }
  for (int i = total + threadIdx.x; i < idx_stride; i += 256) out[i] = -1;
  if (threadIdx.x == 0) pair_cnt[e] = total;
}

// Partial combine of the gather exchange: for every token of the whole batch the weighted sum over those of
// its k pairs whose expert lives on this rank ([exp_lo, exp_hi)), in ascending expert order, separately rounded
// multiply and add from zero (the per-rank prefix of the single-device combine). Tokens without a local expert
// get zeros. Rows of Y are indexed by the global pair id.
__global__ void __launch_bounds__(256) ep_combine_partial_kernel(const float *__restrict__ Y,
                                                                 const int32_t *__restrict__ pair_exp,
                                                                 const float *__restrict__ pair_w, int exp_lo,
                                                                 int exp_hi, float *__restrict__ out, int H, int k) {
  const int t = blockIdx.x;
  __shared__ int s_row[8];
  __shared__ float s_w[8];
  __shared__ int s_n;
  if (threadIdx.x == 0) {
    int ex[8], ord[8], n = 0;
    for (int s = 0; s < k; ++s) {
      const int e = pair_exp[t * k + s];
      if (e >= exp_lo && e < exp_hi) { ex[n] = e; ord[n] = s; ++n; }
    }
    for (int a = 1; a < n; ++a) {  // insertion sort by expert id
      const int o = ord[a], eo = ex[a];
      int b = a - 1;
      while (b >= 0 && ex[b] > eo) { ord[b + 1] = ord[b]; ex[b + 1] = ex[b]; --b; }
      ord[b + 1] = o;
      ex[b + 1] = eo;
    }
    for (int s = 0; s < n; ++s) {
      s_row[s] = t * k + ord[s];
      s_w[s] = pair_w[t * k + ord[s]];
    }
    s_n = n;
  }
  __syncthreads();
  const int n = s_n;
  for (int h = threadIdx.x * 4; h < H; h += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < n; ++s) {
      const float4 y = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)s_row[s] * H + h));
      const float w = s_w[s];
      acc.x = __fadd_rn(acc.x, __fmul_rn(w, y.x));
      acc.y = __fadd_rn(acc.y, __fmul_rn(w, y.y));
      acc.z = __fadd_rn(acc.z, __fmul_rn(w, y.z));
      acc.w = __fadd_rn(acc.w, __fmul_rn(w, y.w));
    }
    *reinterpret_cast<float4 *>(out + (size_t)t * H + h) = acc;
  }
}

// Sum of the per-rank partial rows in ascending rank order (experts are contiguous per rank, so this is the
// single-device expert order with the additions regrouped per rank), then the optional residual, then the store.
template <int ODT>
__global__ void __launch_bounds__(256) ep_reduce_kernel(const float *__restrict__ parts, int n_ranks, int64_t rank_stride,
                                                        const void *__restrict__ resid, int resid_dtype, void *__restrict__ out,
                                                        int64_t n4) {
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
    float4 acc = __ldg(reinterpret_cast<const float4 *>(parts) + i);
    for (int r = 1; r < n_ranks; ++r) {
      const float4 v = __ldg(reinterpret_cast<const float4 *>(parts + r * rank_stride) + i);
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    float r4[4] = {acc.x, acc.y, acc.z, acc.w};
    if (resid) {
#pragma unroll
      for (int j = 0; j < 4; ++j) r4[j] = __fadd_rn(load_as_f32(resid, resid_dtype, i * 4 + j), r4[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) store_from_f32(out, ODT, i * 4 + j, r4[j]);
  }
}

// ---- "peer" exchange: the same two steps with the rows moved by this library's own kernels over NVLink peer
// mappings (every rank maps every other rank's exchange buffers into its address space).

// dst[r * bytes_per_rank + i] = src[r][i]: pulls the published rows (or routing tables) of every rank into
// local memory, 16 bytes per thread and step; source r == own rank is a local copy.
__global__ void __launch_bounds__(256) ep_peer_gather_kernel(const uint4 *const *__restrict__ src, int n_ranks,
                                                             int64_t u4_per_rank, uint4 *__restrict__ dst) {
  const int64_t total = (int64_t)n_ranks * u4_per_rank;
  const int64_t stride = (int64_t)gridDim.x * blockDim.x;
  // four independent peer loads in flight per thread: NVLink latency is a few microseconds
  for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += 4 * stride) {
    uint4 v[4];
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t idx = i + u * stride;
      if (idx < total) {
        const int r = (int)(idx / u4_per_rank);
        v[u] = src[r][idx - (int64_t)r * u4_per_rank];
      }
    }
#pragma unroll
    for (int u = 0; u < 4; ++u) {
      const int64_t idx = i + u * stride;
      if (idx < total) dst[idx] = v[u];
    }
  }
}

// ep_combine_partial with the result row stored straight into the token owner's buffer: parts[owner] points at
// the owner's [n_ranks][T_loc][H] f32 array, this rank fills slot `my_rank`. Tokens without a local expert are
// skipped (the owner knows from its own routing table which ranks contribute).
__global__ void __launch_bounds__(256) ep_combine_partial_peer_kernel(const float *__restrict__ Y,
                                                                      const int32_t *__restrict__ pair_exp,
                                                                      const float *__restrict__ pair_w, int exp_lo,
                                                                      int exp_hi, float *const *__restrict__ parts,
                                                                      int my_rank, int T_loc, int T, int H, int k,
                                                                      int64_t parts_off, float *__restrict__ stage) {
  // one warp per token: lanes 0..k-1 hold the token's slots, the local ones are ranked by expert id
  // The grid walks the tokens starting with those of the next higher rank: at any moment every rank is sending
  // to a different owner instead of all ranks to the same one.
  const int lane = threadIdx.x & 31;
  int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  t += ((my_rank + 1) * T_loc) % T;
  if (t >= T) t -= T;
  const int e = lane < k ? pair_exp[t * k + lane] : -1;
  const float w = lane < k ? pair_w[t * k + lane] : 0.f;
  const bool mine = lane < k && e >= exp_lo && e < exp_hi;
  const unsigned m = __ballot_sync(0xffffffffu, mine);
  const int n = __popc(m);
  if (n == 0) return;
  int rank = 0;
  for (int j = 0; j < k; ++j) {
    const int ej = __shfl_sync(0xffffffffu, e, j);
    if (((m >> j) & 1u) && ej < e) ++rank;
  }
  int row[8];
  float ws[8];
#pragma unroll
  for (int sl = 0; sl < 8; ++sl) {
    const unsigned b = __ballot_sync(0xffffffffu, mine && rank == sl);
    const int src = b ? __ffs(b) - 1 : 0;
    row[sl] = t * k + src;
    ws[sl] = __shfl_sync(0xffffffffu, w, src);
  }
  const int owner = t / T_loc;
  float *out = (stage && owner != my_rank) ? stage + (size_t)t * H  // staged by owner for a later block copy
                                           : parts[owner] + parts_off + ((size_t)my_rank * T_loc + (t % T_loc)) * H;
  for (int h = lane * 4; h < H; h += 128) {
    float4 y[8];
#pragma unroll
    for (int sl = 0; sl < 8; ++sl)
      if (sl < n) y[sl] = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)row[sl] * H + h));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int sl = 0; sl < 8; ++sl) {
      if (sl < n) {
        acc.x = __fadd_rn(acc.x, __fmul_rn(ws[sl], y[sl].x));
        acc.y = __fadd_rn(acc.y, __fmul_rn(ws[sl], y[sl].y));
        acc.z = __fadd_rn(acc.z, __fmul_rn(ws[sl], y[sl].z));
        acc.w = __fadd_rn(acc.w, __fmul_rn(ws[sl], y[sl].w));
      }
    }
    *reinterpret_cast<float4 *>(out + h) = acc;
  }
}

// Sum over the ranks that own at least one of the token's k experts, ascending rank (the others wrote nothing).
template <int ODT>
__global__ void __launch_bounds__(256) ep_reduce_sel_kernel(const float *__restrict__ parts, int n_ranks, int T_loc,
                                                            const int32_t *__restrict__ pair_exp, int k, int e_loc,
                                                            const void *__restrict__ resid, int resid_dtype,
                                                            void *__restrict__ out, int H) {
  const int t = blockIdx.x;
  unsigned long long mask = 0;
  for (int s = 0; s < k; ++s) mask |= 1ull << (pair_exp[t * k + s] / e_loc);
  for (int h = threadIdx.x * 4; h < H; h += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int r = 0; r < n_ranks; ++r) {
      if (!((mask >> r) & 1ull)) continue;
      const float4 v = __ldg(reinterpret_cast<const float4 *>(parts + ((size_t)r * T_loc + t) * H + h));
      acc.x = __fadd_rn(acc.x, v.x);
      acc.y = __fadd_rn(acc.y, v.y);
      acc.z = __fadd_rn(acc.z, v.z);
      acc.w = __fadd_rn(acc.w, v.w);
    }
    float r4[4] = {acc.x, acc.y, acc.z, acc.w};
    if (resid) {
#pragma unroll
      for (int j = 0; j < 4; ++j) r4[j] = __fadd_rn(load_as_f32(resid, resid_dtype, (int64_t)t * H + h + j), r4[j]);
    }
#pragma unroll
    for (int j = 0; j < 4; ++j) store_from_f32(out, ODT, (int64_t)t * H + h + j, r4[j]);
  }
}

// ep_combine_partial_peer with the row stored as fp16 under a per-row power-of-two scale (half the bytes over
// NVLink): the row's slot keeps its f32 stride, the first 2H bytes hold the scaled halves and the float at element
// H/2 the inverse scale. The sum itself is formed in f32 exactly as above; only its stored form is rounded (2^-11
// relative to the row's largest element). H <= 2048, a multiple of 256; lane l covers elements 256 it + 8 l .. + 7.
__global__ void __launch_bounds__(256) ep_combine_partial_peer_f16_kernel(const float *__restrict__ Y,
                                                                          const int32_t *__restrict__ pair_exp,
                                                                          const float *__restrict__ pair_w, int exp_lo,
                                                                          int exp_hi, float *const *__restrict__ parts,
                                                                          int my_rank, int T_loc, int T, int H, int k,
                                                                          int64_t parts_off) {
  const int lane = threadIdx.x & 31;
  int t = blockIdx.x * 8 + (threadIdx.x >> 5);
  if (t >= T) return;
  t += ((my_rank + 1) * T_loc) % T;
  if (t >= T) t -= T;
  const int e = lane < k ? pair_exp[t * k + lane] : -1;
  const float w = lane < k ? pair_w[t * k + lane] : 0.f;
  const bool mine = lane < k && e >= exp_lo && e < exp_hi;
  const unsigned m = __ballot_sync(0xffffffffu, mine);
  const int n = __popc(m);
  if (n == 0) return;
  int rank = 0;
  for (int j = 0; j < k; ++j) {
    const int ej = __shfl_sync(0xffffffffu, e, j);
    if (((m >> j) & 1u) && ej < e) ++rank;
  }
  int row[8];
  float ws[8];
#pragma unroll
  for (int sl = 0; sl < 8; ++sl) {
    const unsigned b = __ballot_sync(0xffffffffu, mine && rank == sl);
    const int src = b ? __ffs(b) - 1 : 0;
    row[sl] = t * k + src;
    ws[sl] = __shfl_sync(0xffffffffu, w, src);
  }
  const int nit = H >> 8;
  float acc[8][8];
  float amax = 0.f;
#pragma unroll
  for (int it = 0; it < 8; ++it) {
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[it][j] = 0.f;
    if (it < nit) {
      const int h = 256 * it + 8 * lane;
#pragma unroll
      for (int sl = 0; sl < 8; ++sl) {
        if (sl < n) {
          const float4 a = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)row[sl] * H + h));
          const float4 b = __ldg(reinterpret_cast<const float4 *>(Y + (size_t)row[sl] * H + h + 4));
          const float y[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[it][j] = __fadd_rn(acc[it][j], __fmul_rn(ws[sl], y[j]));
        }
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) amax = fmaxf(amax, fabsf(acc[it][j]));
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  // power-of-two scale that puts the largest magnitude in [2^14, 2^15); an all-zero, infinite or NaN row keeps 1
  const int be = (int)((__float_as_uint(amax) >> 23) & 0xffu);
  int ex = 0;
  if (be != 0 && be != 0xff) ex = max(-100, min(100, 141 - be));
  const float scale = __uint_as_float((uint32_t)(ex + 127) << 23), inv = __uint_as_float((uint32_t)(127 - ex) << 23);
  float *slot = parts[t / T_loc] + parts_off + ((size_t)my_rank * T_loc + (t % T_loc)) * H;
  __half *out = reinterpret_cast<__half *>(slot);
#pragma unroll
  for (int it = 0; it < 8; ++it) {
    if (it < nit) {
      uint32_t o[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h2 = __floats2half2_rn(fminf(fmaxf(acc[it][2 * j] * scale, -65504.f), 65504.f),
                                             fminf(fmaxf(acc[it][2 * j + 1] * scale, -65504.f), 65504.f));
        o[j] = *reinterpret_cast<const uint32_t *>(&h2);
      }
      *reinterpret_cast<uint4 *>(out + 256 * it + 8 * lane) = make_uint4(o[0], o[1], o[2], o[3]);
    }
  }
  if (lane == 0) slot[H / 2] = inv;
}

// ep_reduce_sel over slots written by ep_combine_partial_peer_f16_kernel
template <int ODT>
__global__ void __launch_bounds__(256) ep_reduce_sel_f16_kernel(const float *__restrict__ parts, int n_ranks, int T_loc,
                                                                const int32_t *__restrict__ pair_exp, int k, int e_loc,
                                                                const void *__restrict__ resid, int resid_dtype,
                                                                void *__restrict__ out, int H) {
  const int t = blockIdx.x;
  unsigned long long mask = 0;
  for (int s = 0; s < k; ++s) mask |= 1ull << (pair_exp[t * k + s] / e_loc);
  for (int h = threadIdx.x * 8; h < H; h += 2048) {
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = 0.f;
    for (int r = 0; r < n_ranks; ++r) {
      if (!((mask >> r) & 1ull)) continue;
      const float *slot = parts + ((size_t)r * T_loc + t) * H;
      const float inv = __ldg(slot + H / 2);
      const uint4 v = __ldg(reinterpret_cast<const uint4 *>(reinterpret_cast<const __half *>(slot) + h));
      const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const __half2 h2 = *reinterpret_cast<const __half2 *>(&u[j]);
        acc[2 * j] = __fadd_rn(acc[2 * j], __low2float(h2) * inv);
        acc[2 * j + 1] = __fadd_rn(acc[2 * j + 1], __high2float(h2) * inv);
      }
    }
    if (resid) {
#pragma unroll
      for (int j = 0; j < 8; ++j) acc[j] = __fadd_rn(load_as_f32(resid, resid_dtype, (int64_t)t * H + h + j), acc[j]);
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) store_from_f32(out, ODT, (int64_t)t * H + h + j, acc[j]);
  }
}

}  // namespace

extern "C" {

int knj_ep_peer_gather_launch(const void *const *src_ptrs, int n_ranks, int64_t bytes_per_rank, void *dst, knj_stream_t s) {
  KNJ_REQUIRE(src_ptrs && dst, "knj_ep_peer_gather: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && bytes_per_rank >= 0 && bytes_per_rank % 16 == 0 && aligned16(dst),
              "knj_ep_peer_gather: sizes must be 16-byte multiples at 16-byte aligned bases");
  if (bytes_per_rank == 0) return KNJ_OK;
  const int64_t total = (int64_t)n_ranks * (bytes_per_rank / 16);
  const int64_t blocks = (total + 255) / 256, cap = (int64_t)sm_count() * 8;
  ep_peer_gather_kernel<<<(unsigned)(blocks < cap ? blocks : cap), 256, 0, as_stream(s)>>>(
      reinterpret_cast<const uint4 *const *>(src_ptrs), n_ranks, bytes_per_rank / 16, static_cast<uint4 *>(dst));
  return launch_status("ep_peer_gather_kernel");
}

}  // extern "C"

// the same with every owner's array entered at element `parts_off` (one chunk of a chunked step); with `stage`
// (f32 [T][H], local) the rows of other ranks' tokens go there, in token order = one dense block per owner
int knj::ep_combine_partial_peer_at(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k, int exp_lo,
                                    int exp_hi, float *const *parts_ptrs, int64_t parts_off, float *stage, int my_rank, int T_loc,
                                    cudaStream_t s) {
  KNJ_REQUIRE(Y && pair_exp && pair_w && parts_ptrs, "knj_ep_combine_partial_peer: null pointer");
  KNJ_REQUIRE(k >= 1 && k <= 8 && H > 0 && H % 4 == 0 && exp_lo <= exp_hi && T_loc >= 1 && my_rank >= 0 && parts_off % 4 == 0,
              "knj_ep_combine_partial_peer: bad k / H / expert range / rank");
  if (T <= 0) return KNJ_OK;
  ep_combine_partial_peer_kernel<<<(T + 7) / 8, 256, 0, s>>>(Y, pair_exp, pair_w, exp_lo, exp_hi, parts_ptrs, my_rank, T_loc, T, H, k, parts_off, stage);
  return launch_status("ep_combine_partial_peer_kernel");
}

// fp16 form of the partial rows (see the kernels): H <= 2048, a multiple of 256
int knj::ep_combine_partial_peer_f16_at(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k, int exp_lo,
                                        int exp_hi, float *const *parts_ptrs, int64_t parts_off, int my_rank, int T_loc, cudaStream_t s) {
  KNJ_REQUIRE(Y && pair_exp && pair_w && parts_ptrs, "knj_ep_combine_partial_peer: null pointer");
  KNJ_REQUIRE(k >= 1 && k <= 8 && H > 0 && H % 256 == 0 && H <= 2048 && exp_lo <= exp_hi && T_loc >= 1 && my_rank >= 0 && parts_off % 4 == 0,
              "knj_ep_combine_partial_peer (fp16 rows): bad k / H / expert range / rank");
  if (T <= 0) return KNJ_OK;
  ep_combine_partial_peer_f16_kernel<<<(T + 7) / 8, 256, 0, s>>>(Y, pair_exp, pair_w, exp_lo, exp_hi, parts_ptrs, my_rank, T_loc, T, H, k, parts_off);
  return launch_status("ep_combine_partial_peer_f16_kernel");
}

int knj::ep_reduce_sel_f16(const float *parts, int n_ranks, int T_loc, int H, const int32_t *pair_exp, int k, int experts_per_rank,
                           const void *resid, int resid_dtype, void *out, int out_dtype, cudaStream_t s) {
  KNJ_REQUIRE(parts && pair_exp && out, "knj_ep_reduce_sel: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && n_ranks <= 64 && H > 0 && H % 256 == 0 && H <= 2048 && k >= 1 && k <= 8 && experts_per_rank >= 1,
              "knj_ep_reduce_sel (fp16 rows): bad sizes");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_ep_reduce_sel: out must be f32 or bf16");
  if (T_loc <= 0) return KNJ_OK;
  if (out_dtype == KNJ_DT_F32)
    ep_reduce_sel_f16_kernel<KNJ_DT_F32><<<T_loc, 256, 0, s>>>(parts, n_ranks, T_loc, pair_exp, k, experts_per_rank, resid, resid_dtype, out, H);
  else
    ep_reduce_sel_f16_kernel<KNJ_DT_BF16><<<T_loc, 256, 0, s>>>(parts, n_ranks, T_loc, pair_exp, k, experts_per_rank, resid, resid_dtype, out, H);
  return launch_status("ep_reduce_sel_f16_kernel");
}

extern "C" {

int knj_ep_combine_partial_peer_launch(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k,
                                       int exp_lo, int exp_hi, float *const *parts_ptrs, int my_rank, int T_loc,
                                       knj_stream_t s) {
  return knj::ep_combine_partial_peer_at(Y, pair_exp, pair_w, T, H, k, exp_lo, exp_hi, parts_ptrs, 0, nullptr, my_rank, T_loc, as_stream(s));
}

int knj_ep_reduce_sel_launch(const float *parts, int n_ranks, int T_loc, int H, const int32_t *pair_exp, int k,
                             int experts_per_rank, const void *resid, int resid_dtype, void *out, int out_dtype,
                             knj_stream_t s) {
  KNJ_REQUIRE(parts && pair_exp && out, "knj_ep_reduce_sel: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && n_ranks <= 64 && H > 0 && H % 4 == 0 && k >= 1 && k <= 8 && experts_per_rank >= 1,
              "knj_ep_reduce_sel: bad sizes");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_ep_reduce_sel: out must be f32 or bf16");
  KNJ_REQUIRE(!resid || (resid_dtype >= KNJ_DT_F32 && resid_dtype <= KNJ_DT_F16), "knj_ep_reduce_sel: unknown residual dtype");
  if (T_loc <= 0) return KNJ_OK;
  if (out_dtype == KNJ_DT_F32)
    ep_reduce_sel_kernel<KNJ_DT_F32><<<T_loc, 256, 0, as_stream(s)>>>(parts, n_ranks, T_loc, pair_exp, k, experts_per_rank, resid, resid_dtype, out, H);
  else
    ep_reduce_sel_kernel<KNJ_DT_BF16><<<T_loc, 256, 0, as_stream(s)>>>(parts, n_ranks, T_loc, pair_exp, k, experts_per_rank, resid, resid_dtype, out, H);
  return launch_status("ep_reduce_sel_kernel");
}

int knj_ep_combine_partial_launch(const float *Y, const int32_t *pair_exp, const float *pair_w, int T, int H, int k,
                                  int exp_lo, int exp_hi, float *out, knj_stream_t s) {
  KNJ_REQUIRE(Y && pair_exp && pair_w && out, "knj_ep_combine_partial: null pointer");
  KNJ_REQUIRE(k >= 1 && k <= 8 && H > 0 && H % 4 == 0 && exp_lo <= exp_hi, "knj_ep_combine_partial: bad k / H / expert range");
  if (T <= 0) return KNJ_OK;
  ep_combine_partial_kernel<<<T, 256, 0, as_stream(s)>>>(Y, pair_exp, pair_w, exp_lo, exp_hi, out, H, k);
  return launch_status("ep_combine_partial_kernel");
}

int knj_ep_reduce_launch(const float *parts, int n_ranks, int64_t rank_stride, int T, int H, const void *resid,
                         int resid_dtype, void *out, int out_dtype, knj_stream_t s) {
  KNJ_REQUIRE(parts && out, "knj_ep_reduce: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && H > 0 && H % 4 == 0 && rank_stride % 4 == 0, "knj_ep_reduce: bad sizes");
  KNJ_REQUIRE(out_dtype == KNJ_DT_F32 || out_dtype == KNJ_DT_BF16, "knj_ep_reduce: out must be f32 or bf16");
  KNJ_REQUIRE(!resid || (resid_dtype >= KNJ_DT_F32 && resid_dtype <= KNJ_DT_F16), "knj_ep_reduce: unknown residual dtype");
  if (T <= 0) return KNJ_OK;
  const int64_t n4 = (int64_t)T * H / 4;
  const int64_t blocks = (n4 + 255) / 256, cap = (int64_t)sm_count() * 16;
  const unsigned grid = (unsigned)(blocks < cap ? blocks : cap);
  if (out_dtype == KNJ_DT_F32)
    ep_reduce_kernel<KNJ_DT_F32><<<grid, 256, 0, as_stream(s)>>>(parts, n_ranks, rank_stride, resid, resid_dtype, out, n4);
  else
    ep_reduce_kernel<KNJ_DT_BF16><<<grid, 256, 0, as_stream(s)>>>(parts, n_ranks, rank_stride, resid, resid_dtype, out, n4);
  return launch_status("ep_reduce_kernel");
}

int knj_ep_pack_launch(const void *x, int row_bytes, int top_k, const int32_t *pair_idx, int idx_stride,
                       const int32_t *pair_cnt, int E, int32_t *send_off, void *send_rows, int32_t *pair_row,
                       knj_stream_t s) {
  KNJ_REQUIRE(x && pair_idx && pair_cnt && send_off && send_rows && pair_row, "knj_ep_pack: null pointer");
  KNJ_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && aligned16(x) && aligned16(send_rows),
              "knj_ep_pack: rows must be 16-byte multiples at 16-byte aligned bases");
  KNJ_REQUIRE(E >= 1 && E <= 256 && top_k >= 1, "knj_ep_pack: bad expert count / top_k");
  ep_offsets_kernel<<<1, 256, 0, as_stream(s)>>>(pair_cnt, E, send_off);
  int rc = launch_status("ep_offsets_kernel");
  if (rc) return rc;
  dim3 grid(64, E);
  ep_pack_kernel<<<grid, 256, 0, as_stream(s)>>>(static_cast<const uint4 *>(x), row_bytes / 16, top_k, pair_idx,
                                                 idx_stride, pair_cnt, send_off, E, static_cast<uint4 *>(send_rows),
                                                 pair_row);
  return launch_status("ep_pack_kernel");
}

int knj_ep_plan_launch(const int32_t *counts, int n_ranks, int n_local_experts, int idx_stride, int32_t *pair_idx,
                       int32_t *pair_cnt, int32_t *exp_list, int32_t *n_active, knj_stream_t s) {
  KNJ_REQUIRE(counts && pair_idx && pair_cnt && exp_list && n_active, "knj_ep_plan: null pointer");
  KNJ_REQUIRE(n_ranks >= 1 && n_ranks <= 64 && n_local_experts >= 1 && idx_stride >= 1, "knj_ep_plan: bad sizes");
  ep_plan_kernel<<<n_local_experts, 256, 0, as_stream(s)>>>(counts, n_ranks, n_local_experts, idx_stride, pair_idx,
                                                            pair_cnt);
  int rc = launch_status("ep_plan_kernel");
  if (rc) return rc;
  return knj_active_list_launch(pair_cnt, n_local_experts, exp_list, n_active, s);
}

}  // extern "C"
