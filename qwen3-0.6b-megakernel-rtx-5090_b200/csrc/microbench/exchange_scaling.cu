// Stand-alone microbenchmark: (1) time of one all-to-all round of tagged 8-byte words versus the number of
// participating CTAs and of copies of the buffer; (2) per-SM cp.async.bulk bandwidth versus the number of SMs
// that stream.  Every spin is bounded.  Build and run:
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o exchange_scaling exchange_scaling.cu && ./exchange_scaling
// Results on B200: profiles/primitives_b200.md
#include <cuda_runtime.h>
#include <stdio.h>
#include <stdint.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)
__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) { unsigned long long w; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory"); return w; }
__device__ __forceinline__ void ll_store(unsigned long long *p, unsigned long long w) { asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory"); }
__global__ void k_exchange(unsigned long long *buf, int nwords, int R, int rounds, long long *out, int *err) {
  const int ncta = gridDim.x, cta = blockIdx.x, tid = threadIdx.x;
  const int r0 = (int)(((long long)nwords * cta) / ncta), r1 = (int)(((long long)nwords * (cta + 1)) / ncta);
  __shared__ float sink[4096];
  const size_t rep_stride = 4096, par_stride = rep_stride * 8;
  const int mine = cta % R;
  long long t0 = clock64();
  for (int r = 1; r <= rounds; ++r) {
    unsigned long long *b = buf + (r & 1) * par_stride;
    for (int row = r0 + tid; row < r1; row += blockDim.x)   // coalesced: thread = word
      for (int k = 0; k < R; ++k) ll_store(b + k * rep_stride + row, ((unsigned long long)r << 32) | (unsigned)row);
    const unsigned long long *rb = b + mine * rep_stride;
    for (int i = tid; i < nwords; i += blockDim.x) {
      unsigned long long w = ll_load(rb + i); long long spins = 0;
      while ((unsigned)(w >> 32) != (unsigned)r) { w = ll_load(rb + i); if (++spins > 2000000) { *err = 1; break; } }
      sink[i] = __uint_as_float((unsigned)w);
    }
    __syncthreads();
  }
  if (tid == 0) out[cta] = (clock64() - t0) / rounds;
}
constexpr int NS = 20, SB = 8192;
__global__ void k_stream(const unsigned char *src, size_t per_cta, int iters, long long *out) {
  extern __shared__ __align__(128) unsigned char smem[];
  uint64_t *full = (uint64_t *)(smem + NS * SB);
  if (threadIdx.x == 0) {
    for (int i = 0; i < NS; ++i) asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(s32(full + i)));
    asm volatile("fence.mbarrier_init.release.cluster;");
    const unsigned char *p = src + (size_t)blockIdx.x * per_cta; size_t off = 0; uint32_t phase = 0;
    long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
      for (int i = 0; i < NS; ++i) {
        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(s32(full + i)), "r"(SB) : "memory");
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(s32(smem + i * SB)), "l"(p + off), "r"(SB), "r"(s32(full + i)) : "memory");
        off += SB; if (off + SB > per_cta) off = 0;
      }
      for (int i = 0; i < NS; ++i) { uint32_t ok = 0; int g = 0; while (!ok && ++g < 4000000) asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2; selp.u32 %0,1,0,p; }" : "=r"(ok) : "r"(s32(full + i)), "r"(phase) : "memory"); }
      phase ^= 1;
    }
    out[blockIdx.x] = clock64() - t0;
  }
}
int main() {
  cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, 0)); int nsm = prop.multiProcessorCount;
  long long *out; CK(cudaMallocManaged(&out, 4096 * 8)); int *err; CK(cudaMallocManaged(&err, 4)); *err = 0;
  unsigned long long *buf; size_t words = 2ull * 8 * 4096; CK(cudaMalloc(&buf, words * 8));
  int grids[6] = {16, 32, 48, 64, 96, 148}; int nws[2] = {1024, 3072}; int Rs[2] = {1, 4};
  for (int n : nws) for (int R : Rs) for (int g : grids) {
    CK(cudaMemset(buf, 0, words * 8)); int rounds = 300;
    void *args[] = {&buf, &n, &R, &rounds, &out, &err};
    CK(cudaLaunchCooperativeKernel((void *)k_exchange, dim3(g), dim3(512), args, 0, 0)); CK(cudaDeviceSynchronize());
    long long sum = 0; for (int i = 0; i < g; ++i) sum += out[i];
    printf("exchange %4d words R=%d grid %3d: %.2f us/round (err %d)\n", n, R, g, sum / g / 1965.0, *err);
  }
  size_t per_cta = 4u << 20; unsigned char *src; CK(cudaMalloc(&src, per_cta * nsm)); CK(cudaMemset(src, 1, per_cta * nsm));
  CK(cudaFuncSetAttribute(k_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, NS * SB + 256));
  for (int g : grids) {
    int iters = 100;  // 100 * 160 KB = 16 MB per CTA, wraps within its 4 MB region -> L2 resident after first pass for small g
    k_stream<<<g, 32, NS * SB + 256>>>(src, per_cta, iters, out); CK(cudaDeviceSynchronize());
    long long mx = 0; for (int i = 0; i < g; ++i) if (out[i] > mx) mx = out[i];
    double sec = mx / 1.965e9, bytes = (double)iters * NS * SB;
    printf("stream grid %3d (4 MB region per CTA, re-read): %.1f GB/s per SM, %.2f TB/s total\n", g, bytes / sec / 1e9, bytes * g / sec / 1e12);
  }
  return 0;
}
