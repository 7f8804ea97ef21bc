/* knj_index.h -- thread / block index helpers with the reference's names
 * (kernels/knj_index.h: knj_tid :63, knj_bid :67, knj_gid :73). The reference
 * needs them because its device runtime is linked without a grid-size query;
 * CUDA has threadIdx/blockIdx, so these are one-liners. Kernels that mirror a
 * reference kernel still take (n_threads, n_blocks) as explicit arguments. */
#ifndef KNJ_INDEX_H
#define KNJ_INDEX_H

#if defined(__CUDACC__)
__device__ __forceinline__ unsigned knj_tid(void) { return threadIdx.x; }
__device__ __forceinline__ unsigned knj_bid(void) { return blockIdx.x; }
__device__ __forceinline__ unsigned knj_gid(unsigned threads_per_block, unsigned blocks) {
  (void)blocks;
  return blockIdx.x * threads_per_block + threadIdx.x;
}
#endif

#endif /* KNJ_INDEX_H */
