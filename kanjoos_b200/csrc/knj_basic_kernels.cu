// knj_basic_kernels.cu -- sm_100a versions of the four kernels of the
// reference's kernels/knj_kernels.hip (control, capability probe, W4-g128 x int8
// GEMM, Asum builder) and the Q4_K / Q6_K verification decoders.
#include "knj_common.cuh"
#include "knj_dot.h"
#include "knj_index.h"
#include "knj_pack.h"
#include "knj_q4k.h"

using namespace knj;

// ---------------------------------------------------------------------------
// knj_control: a value the host can predict from the launch arguments alone.
// ---------------------------------------------------------------------------
extern "C" __global__ void knj_control(uint32_t *out, uint32_t seed, uint32_t n_threads, uint32_t n_blocks) {
  if (knj_gid(n_threads, n_blocks) == 0u) {
    out[0] = seed + 1u;
    out[1] = n_blocks;
  }
}

// ---------------------------------------------------------------------------
// knj_probe_caps: capabilities verified by executing them (one warp).
// ---------------------------------------------------------------------------
extern "C" __global__ void knj_probe_caps(uint32_t *cap, const int32_t *in) {
  __shared__ __align__(16) uint32_t landing[4];
  __shared__ uint64_t bar;
  const unsigned lane = threadIdx.x & 31u;

  // (a) bulk async copy + mbarrier transaction count, bounded wait. The source
  // is the first 16 bytes of `cap` as the host left them.
  uint32_t before[4] = {0, 0, 0, 0};
  bool copy_ok = false;
  if (lane == 0) {
    for (int i = 0; i < 4; ++i) before[i] = cap[i];
    mbar_init(&bar, 1);
    mbar_init_fence();
  }
  __syncwarp();
  if (lane == 0) {
    mbar_expect_tx(&bar, 16);
    bulk_g2s(landing, cap, 16, &bar);
    if (mbar_wait(&bar, 0)) {
      copy_ok = true;
      for (int i = 0; i < 4; ++i) copy_ok = copy_ok && landing[i] == before[i];
    }
  }
  __syncwarp();

  // (b) fp16 tensor-core MMA over 4-bit integers stored as fp16 SUBNORMAL bit
  // patterns (0x000q = q * 2^-24): every lane feeds codes derived from its
  // lane id; the expected sums are small integers, so the check is exact.
  bool mma_ok;
  {
    const unsigned g = lane >> 2, t = lane & 3u;
    // A[row][k] = (row + k) & 15 ; B[k][col] = ((k * (col + 1)) % 7) - 3
    auto a_code = [](unsigned row, unsigned k) { return (row + k) & 15u; };
    auto b_val = [](unsigned k, unsigned col) { return (float)((int)((k * (col + 1u)) % 7u) - 3); };
    auto pack_a = [&](unsigned row, unsigned k) { return a_code(row, k) | (a_code(row, k + 1) << 16); };
    auto pack_b = [&](unsigned k, unsigned col) {
      const __half2 h = __floats2half2_rn(b_val(k, col), b_val(k + 1, col));
      return *reinterpret_cast<const uint32_t *>(&h);
    };
    float d[4] = {0.f, 0.f, 0.f, 0.f};
    mma_f16_16816(d, pack_a(g, 2 * t), pack_a(g + 8, 2 * t), pack_a(g, 2 * t + 8), pack_a(g + 8, 2 * t + 8),
                  pack_b(2 * t, g), pack_b(2 * t + 8, g));
    bool ok = true;
    for (int i = 0; i < 4; ++i) {
      const unsigned row = g + ((i & 2) ? 8u : 0u), col = 2 * t + (i & 1);
      float want = 0.f;
      for (unsigned k = 0; k < 16; ++k) want += (float)a_code(row, k) * b_val(k, col);
      ok = ok && (d[i] * 16777216.0f == want);
    }
    mma_ok = __all_sync(0xffffffffu, ok);
  }

  if (knj_gid(32u, 1u) != 0u) return;

  // integer dot identity
  int d4 = 0;
  d4 = knj_dot4_i32_i8(0x01010101, 0x01010101, d4);
  cap[0] = (d4 == 4) ? 1u : 0u;

  // packed fp16 fma: two chained 1*1 + acc from an explicitly zeroed accumulator
  {
    const __half2 one = __floats2half2_rn(1.0f, 1.0f);
    __half2 r = __floats2half2_rn(0.0f, 0.0f);
    r = __hfma2(one, one, r);
    r = __hfma2(one, one, r);
    const uint32_t bits = *reinterpret_cast<const uint32_t *>(&r);
    cap[1] = ((bits & 0xffffu) == 0x4000u) ? 1u : 0u;
    cap[4] = bits & 0xffffu;
  }
  cap[2] = 1u;
  cap[3] = in ? (uint32_t)in[0] : 0u;
  cap[5] = mma_ok ? 1u : 0u;
  cap[6] = copy_ok ? 1u : 0u;
  cap[7] = 0u;  // TMEM allocation is probed by the prefill kernel's own self-test
}

// ---------------------------------------------------------------------------
// W4-g128 x int8
// ---------------------------------------------------------------------------
__device__ __forceinline__ uint32_t ld_u32_unaligned4(const uint8_t *p) {
  // group bases are 4-byte aligned (68-byte stride from an aligned base)
  return *reinterpret_cast<const uint32_t *>(p);
}

extern "C" __global__ void knj_gemm_w4_i8(const uint8_t *__restrict__ Bq, const uint32_t *__restrict__ Act,
                                          const int32_t *__restrict__ Asum, float *__restrict__ C, uint32_t M,
                                          uint32_t N, uint32_t K, uint32_t n_threads, uint32_t n_blocks) {
  const uint32_t stride = n_threads * n_blocks;
  const uint32_t groups = K / KNJ_GROUP_EXPERT;
  const uint32_t gbytes = KNJ_GROUP_STRIDE_BYTES(4, KNJ_GROUP_EXPERT);
  for (uint32_t idx = knj_gid(n_threads, n_blocks); idx < M * N; idx += stride) {
    const uint32_t m = idx / N, n = idx - m * N;
    const uint8_t *col = Bq + (size_t)n * groups * gbytes;
    const uint2 *arow = reinterpret_cast<const uint2 *>(Act + (size_t)m * (K / 8) * 2);
    float acc = 0.0f;
    for (uint32_t g = 0; g < groups; ++g) {
      const uint8_t *grp = col + (size_t)g * gbytes;
      const float scale = knj_half_bits_to_float(knj_load_u16(grp + 64));
      int raw = 0;
#pragma unroll 4
      for (uint32_t j = 0; j < KNJ_GROUP_EXPERT / 8; ++j) {
        int lo, hi;
        knj_unpack8_u4(ld_u32_unaligned4(grp + 4 * j), &lo, &hi);
        const uint2 a = arow[g * (KNJ_GROUP_EXPERT / 8) + j];
        raw = knj_dot4_i32_i8(lo, (int)a.x, raw);
        raw = knj_dot4_i32_i8(hi, (int)a.y, raw);
      }
      const float centred = __fsub_rn((float)raw, (float)(KNJ_NIBBLE_BIAS * Asum[(size_t)m * groups + g]));
      acc = __fadd_rn(acc, __fmul_rn(scale, centred));
    }
    C[idx] = acc;
  }
}

extern "C" __global__ void knj_build_asum(const uint32_t *__restrict__ Act, int32_t *__restrict__ Asum, uint32_t M,
                                          uint32_t K, uint32_t n_threads, uint32_t n_blocks) {
  const uint32_t stride = n_threads * n_blocks;
  const uint32_t groups = K / KNJ_GROUP_EXPERT;
  for (uint32_t idx = knj_gid(n_threads, n_blocks); idx < M * groups; idx += stride) {
    const uint32_t m = idx / groups, g = idx - m * groups;
    const uint2 *a = reinterpret_cast<const uint2 *>(Act + (size_t)m * (K / 8) * 2) + g * (KNJ_GROUP_EXPERT / 8);
    int s = 0;
#pragma unroll 4
    for (uint32_t j = 0; j < KNJ_GROUP_EXPERT / 8; ++j) {
      const uint2 w = a[j];
      s = knj_dot4_i32_i8(0x01010101, (int)w.x, s);
      s = knj_dot4_i32_i8(0x01010101, (int)w.y, s);
    }
    Asum[idx] = s;
  }
}

// ---------------------------------------------------------------------------
// Q4_K / Q6_K -> f32 (verification only)
// ---------------------------------------------------------------------------
// One thread decodes four consecutive weights of one superblock. The two
// roundings of the CPU decoder (the product d1*q is exact, the subtraction
// rounds once) are reproduced with explicitly non-contracted operations.
__global__ void q4k_dequant_kernel(const uint8_t *__restrict__ blocks, float4 *__restrict__ out, uint64_t n_quads) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_quads;
       i += (uint64_t)gridDim.x * blockDim.x) {
    const uint64_t b = i >> 6;        // 64 quads per superblock
    const int r0 = (int)(i & 63) * 4; // first weight of the quad
    const uint8_t *blk = blocks + b * KNJ_Q4K_BYTES;
    const int j = r0 >> 5;
    uint8_t sc, mn;
    knj_q4k_scale_min(blk + KNJ_Q4K_OFF_SCALE, j, &sc, &mn);
    const float d1 = __fmul_rn(knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_D)), (float)sc);
    const float m1 = __fmul_rn(knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q4K_OFF_DMIN)), (float)mn);
    const uint32_t w = *reinterpret_cast<const uint32_t *>(blk + KNJ_Q4K_OFF_QS + ((j >> 1) << 5) + (r0 & 31));
    const uint32_t nib = (j & 1) ? (w >> 4) : w;
    float4 o;
    o.x = __fsub_rn(__fmul_rn(d1, (float)(nib & 15u)), m1);
    o.y = __fsub_rn(__fmul_rn(d1, (float)((nib >> 8) & 15u)), m1);
    o.z = __fsub_rn(__fmul_rn(d1, (float)((nib >> 16) & 15u)), m1);
    o.w = __fsub_rn(__fmul_rn(d1, (float)((nib >> 24) & 15u)), m1);
    out[i] = o;
  }
}

__global__ void q6k_dequant_kernel(const uint8_t *__restrict__ blocks, float *__restrict__ out, uint64_t n) {
  for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x) {
    const uint8_t *blk = blocks + (i >> 8) * KNJ_Q6K_BYTES;
    const int r = (int)(i & 255);
    const int hf = r >> 7, c = (r >> 5) & 3, l = r & 31;
    const uint32_t lo = blk[KNJ_Q6K_OFF_QL + hf * 64 + ((c & 1) << 5) + l];
    const uint32_t nib = (c & 2) ? (lo >> 4) : (lo & 15u);
    const uint32_t top = ((uint32_t)blk[KNJ_Q6K_OFF_QH + hf * 32 + l] >> (2 * c)) & 3u;
    const int q = (int)(nib | (top << 4)) - 32;
    const float d = knj_half_bits_to_float(knj_load_u16(blk + KNJ_Q6K_OFF_D));
    const float s = (float)((const int8_t *)(blk + KNJ_Q6K_OFF_SC))[hf * 8 + (l >> 4) + 2 * c];
    out[i] = __fmul_rn(__fmul_rn(d, s), (float)q);
  }
}

// The three dot helpers of knj_dot.h executed on the device, one (a, b, acc) triple per thread: lets a test pin
// the device result to the host definition (the reference's device mirrors: tools/bench/gemm_w4.hip:345-397).
__global__ void dot_helpers_kernel(const int32_t *__restrict__ a, const int32_t *__restrict__ b, const int32_t *__restrict__ acc,
                                   int32_t *__restrict__ out4, int32_t *__restrict__ out8, int32_t *__restrict__ out2, int n) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n) return;
  out4[i] = knj_dot4_i32_i8(a[i], b[i], acc[i]);
  out8[i] = knj_dot8_i32_i4(a[i], b[i], acc[i]);
  out2[i] = knj_dot2_i32_i16(a[i], b[i], acc[i]);
}

extern "C" {

int knj_control_launch(uint32_t *out, uint32_t seed, uint32_t n_threads, uint32_t n_blocks, knj_stream_t s) {
  KNJ_REQUIRE(out, "knj_control: null out");
  KNJ_REQUIRE(n_threads >= 1 && n_threads <= 1024 && n_blocks >= 1, "knj_control: bad geometry %u x %u", n_threads,
              n_blocks);
  knj_control<<<n_blocks, n_threads, 0, as_stream(s)>>>(out, seed, n_threads, n_blocks);
  return launch_status("knj_control");
}

int knj_probe_caps_launch(uint32_t *cap, const int32_t *in, knj_stream_t s) {
  KNJ_REQUIRE(cap && aligned16(cap), "knj_probe_caps: cap must be a 16-byte aligned array of 8 words");
  knj_probe_caps<<<1, 32, 0, as_stream(s)>>>(cap, in);
  return launch_status("knj_probe_caps");
}

int knj_build_asum_launch(const uint32_t *Act, int32_t *Asum, uint32_t M, uint32_t K, uint32_t n_threads,
                          uint32_t n_blocks, knj_stream_t s) {
  KNJ_REQUIRE(Act && Asum, "knj_build_asum: null pointer");
  KNJ_REQUIRE(K % KNJ_GROUP_EXPERT == 0 && M > 0, "knj_build_asum: K=%u must be a multiple of 128", K);
  KNJ_REQUIRE(n_threads >= 1 && n_threads <= 1024 && n_blocks >= 1, "knj_build_asum: bad geometry");
  KNJ_REQUIRE((reinterpret_cast<uintptr_t>(Act) & 7u) == 0, "knj_build_asum: Act must be 8-byte aligned");
  knj_build_asum<<<n_blocks, n_threads, 0, as_stream(s)>>>(Act, Asum, M, K, n_threads, n_blocks);
  return launch_status("knj_build_asum");
}

int knj_gemm_w4_i8_launch(const uint8_t *Bq, const uint32_t *Act, const int32_t *Asum, float *C, uint32_t M,
                          uint32_t N, uint32_t K, uint32_t n_threads, uint32_t n_blocks, knj_stream_t s) {
  KNJ_REQUIRE(Bq && Act && Asum && C, "knj_gemm_w4_i8: null pointer");
  KNJ_REQUIRE(K % KNJ_GROUP_EXPERT == 0 && M > 0 && N > 0, "knj_gemm_w4_i8: K=%u must be a multiple of 128", K);
  KNJ_REQUIRE((uint64_t)M * N < (1ull << 32), "knj_gemm_w4_i8: M*N overflows the 32-bit output index");
  KNJ_REQUIRE(n_threads >= 1 && n_threads <= 1024 && n_blocks >= 1, "knj_gemm_w4_i8: bad geometry");
  KNJ_REQUIRE((reinterpret_cast<uintptr_t>(Bq) & 3u) == 0 && (reinterpret_cast<uintptr_t>(Act) & 7u) == 0,
              "knj_gemm_w4_i8: Bq must be 4-byte and Act 8-byte aligned");
  knj_gemm_w4_i8<<<n_blocks, n_threads, 0, as_stream(s)>>>(Bq, Act, Asum, C, M, N, K, n_threads, n_blocks);
  return launch_status("knj_gemm_w4_i8");
}

int knj_q4k_dequant_launch(const uint8_t *blocks, float *out, uint64_t n_blocks, knj_stream_t s) {
  if (n_blocks == 0) return KNJ_OK;
  KNJ_REQUIRE(blocks && out, "knj_q4k_dequant: null pointer");
  KNJ_REQUIRE(aligned16(blocks) && aligned16(out), "knj_q4k_dequant: pointers must be 16-byte aligned");
  const uint64_t quads = n_blocks * 64;
  const unsigned grid = (unsigned)((quads + 255) / 256 < (uint64_t)sm_count() * 16 ? (quads + 255) / 256
                                                                                     : (uint64_t)sm_count() * 16);
  q4k_dequant_kernel<<<grid, 256, 0, as_stream(s)>>>(blocks, reinterpret_cast<float4 *>(out), quads);
  return launch_status("knj_q4k_dequant");
}

int knj_q6k_dequant_launch(const uint8_t *blocks, float *out, uint64_t n_blocks, knj_stream_t s) {
  if (n_blocks == 0) return KNJ_OK;
  KNJ_REQUIRE(blocks && out, "knj_q6k_dequant: null pointer");
  const uint64_t n = n_blocks * 256;
  const unsigned grid = (unsigned)((n + 255) / 256 < (uint64_t)sm_count() * 16 ? (n + 255) / 256
                                                                                 : (uint64_t)sm_count() * 16);
  q6k_dequant_kernel<<<grid, 256, 0, as_stream(s)>>>(blocks, out, n);
  return launch_status("knj_q6k_dequant");
}

int knj_dot_helpers_launch(const int32_t *a, const int32_t *b, const int32_t *acc, int32_t *out4, int32_t *out8,
                           int32_t *out2, int n, knj_stream_t s) {
  KNJ_REQUIRE(a && b && acc && out4 && out8 && out2 && n >= 0, "knj_dot_helpers: null pointer");
  if (n == 0) return KNJ_OK;
  dot_helpers_kernel<<<(n + 255) / 256, 256, 0, as_stream(s)>>>(a, b, acc, out4, out8, out2, n);
  return launch_status("dot_helpers_kernel");
}

}  // extern "C"
