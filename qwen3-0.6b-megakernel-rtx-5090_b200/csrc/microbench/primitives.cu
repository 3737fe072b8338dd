// Microbenchmarks of the primitives the decode megakernel's critical path is made of (stand-alone program):
// timer read cost, L2 load latency (idle and under polling), cross-CTA store->load hop, one all-to-all
// round of tagged 8-byte words over all SMs (polling and flag-based), CTA barrier, fp16 row product from
// shared memory.  Every spin is bounded.  Build and run:
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o primitives primitives.cu && ./primitives
// Results on B200: profiles/primitives_b200.md
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cooperative_groups.h>
#include <stdio.h>
#include <stdint.h>
#include <vector>
namespace cg = cooperative_groups;

#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)

__device__ __forceinline__ unsigned long long ll_load(const unsigned long long *p) {
  unsigned long long w; asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory"); return w;
}
__device__ __forceinline__ void ll_store(unsigned long long *p, unsigned long long w) {
  asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ unsigned long long gtimer() { unsigned long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
__device__ __forceinline__ unsigned smid() { unsigned s; asm volatile("mov.u32 %0, %%smid;" : "=r"(s)); return s; }

// A: timer costs.  out[0] = cycles per clock64, out[1] = cycles per globaltimer read
__global__ void k_timers(long long *out) {
  long long t0 = clock64();
  long long acc = 0;
  for (int i = 0; i < 64; ++i) acc += clock64();
  long long t1 = clock64();
  unsigned long long g = 0;
  for (int i = 0; i < 64; ++i) g += gtimer();
  long long t2 = clock64();
  out[0] = (t1 - t0) / 64; out[1] = (t2 - t1) / 64; out[2] = acc + (long long)g;
}

// B/C: pointer chase in L2 with relaxed.gpu loads (CTA 0 thread 0), optionally while the other CTAs poll `hot`.
__global__ void k_chase(unsigned long long *chain, int n, const unsigned long long *hot, int hot_words, int contend,
                        volatile int *stop, long long *out) {
  if (blockIdx.x == 0) {
    if (threadIdx.x == 0) {
      unsigned long long idx = 0;
      for (int i = 0; i < 64; ++i) idx = ll_load(chain + idx);   // warm
      long long t0 = clock64();
      for (int i = 0; i < n; ++i) idx = ll_load(chain + idx);
      long long t1 = clock64();
      out[0] = (t1 - t0) / n; out[1] = (long long)idx;
      *stop = 1;
      __threadfence();
    }
  } else if (contend) {
    unsigned long long s = 0;
    for (int it = 0; it < 200000; ++it) {
      for (int i = threadIdx.x; i < hot_words; i += blockDim.x) s += ll_load(hot + i);
      if ((it & 7) == 0 && *stop) break;
    }
    if (s == 12345) out[7] = 1;
  }
}

// D: ping-pong between CTA a and CTA b.  out = ns per one-way hop (globaltimer over all rounds)
__global__ void k_pingpong(unsigned long long *words, int a, int b, int rounds, long long *out) {
  if (threadIdx.x != 0) return;
  if (blockIdx.x == a) {
    unsigned long long t0 = gtimer();
    long long c0 = clock64();
    for (int r = 1; r <= rounds; ++r) {
      ll_store(words, r);
      long long spins = 0;
      while (ll_load(words + 16) != (unsigned long long)r) { if (++spins > 4000000) { out[3] = -1; return; } }
    }
    out[0] = (long long)(gtimer() - t0) / (2 * rounds);
    out[1] = (clock64() - c0) / (2 * rounds);
    out[2] = smid();
  } else if (blockIdx.x == b) {
    for (int r = 1; r <= rounds; ++r) {
      long long spins = 0;
      while (ll_load(words) != (unsigned long long)r) { if (++spins > 4000000) { out[3] = -2; return; } }
      ll_store(words + 16, r);
    }
    out[4] = smid();
  }
}

// E: all-to-all exchange round: every CTA stores `per` words (one lane-0 store per warp), then all 512 threads
// poll `nwords` words.  Repeated `rounds` times with tags; two buffers alternate.  out[cta] = cycles per round.
__global__ void k_exchange(unsigned long long *buf, int nwords, int rounds, int sleep_ns, long long *out, int *err) {
  const int ncta = gridDim.x, cta = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = (int)(((long long)nwords * cta) / ncta), r1 = (int)(((long long)nwords * (cta + 1)) / ncta);
  __shared__ float sink[4096];
  long long t0 = clock64();
  for (int r = 1; r <= rounds; ++r) {
    unsigned long long *b = buf + (r & 1) * 4096;
    for (int row = r0 + warp; row < r1; row += 16)
      if (lane == 0) ll_store(b + row, ((unsigned long long)r << 32) | (unsigned)row);
    for (int i = tid; i < nwords; i += blockDim.x) {
      unsigned long long w = ll_load(b + i);
      long long spins = 0;
      while ((unsigned)(w >> 32) != (unsigned)r) {
        if (sleep_ns) __nanosleep(sleep_ns);
        w = ll_load(b + i);
        if (++spins > 2000000) { *err = 1; break; }
      }
      sink[i] = __uint_as_float((unsigned)w);
    }
    __syncthreads();
  }
  long long t1 = clock64();
  if (tid == 0) out[cta] = (t1 - t0) / rounds;
}

// E2: flag-based exchange: data stored plainly (st.cg-like via volatile), then per-CTA flag with release;
// consumers poll 148 flags (acquire) then read data once.
__global__ void k_exchange_flags(float *data, unsigned *flags, int nwords, int rounds, long long *out, int *err) {
  const int ncta = gridDim.x, cta = blockIdx.x, tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int r0 = (int)(((long long)nwords * cta) / ncta), r1 = (int)(((long long)nwords * (cta + 1)) / ncta);
  __shared__ float sink[4096];
  long long t0 = clock64();
  for (int r = 1; r <= rounds; ++r) {
    float *d = data + (r & 1) * 4096;
    unsigned *fl = flags + (r & 1) * 256;
    for (int row = r0 + warp; row < r1; row += 16)
      if (lane == 0) __stcg(d + row, (float)row);
    __syncthreads();
    if (tid == 0) { asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(fl + cta), "r"((unsigned)r) : "memory"); }
    if (tid < ncta) {
      unsigned v; long long spins = 0;
      do { asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(fl + tid) : "memory"); if (++spins > 2000000) { *err = 2; break; } } while (v != (unsigned)r);
    }
    __syncthreads();
    for (int i = tid; i < nwords; i += blockDim.x) sink[i] = __ldcg(d + i);
    __syncthreads();
  }
  long long t1 = clock64();
  if (tid == 0) out[cta] = (t1 - t0) / rounds;
}

// F: barrier and block-sum cost (512 threads).  out[0] = cycles per bar.sync, out[1] = per block_sum
__global__ void k_barrier(long long *out) {
  __shared__ float red[16];
  long long t0 = clock64();
  for (int i = 0; i < 256; ++i) asm volatile("bar.sync 1, 512;" ::: "memory");
  long long t1 = clock64();
  float v = threadIdx.x, tot = 0;
  for (int i = 0; i < 256; ++i) {
    float w = v;
    for (int o = 16; o > 0; o >>= 1) w += __shfl_xor_sync(0xffffffffu, w, o);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = w;
    asm volatile("bar.sync 1, 512;" ::: "memory");
    float t = 0; for (int k = 0; k < 16; ++k) t += red[k];
    tot += t; v += 1.f;
    asm volatile("bar.sync 1, 512;" ::: "memory");
  }
  long long t2 = clock64();
  if (threadIdx.x == 0) { out[0] = (t1 - t0) / 256; out[1] = (t2 - t1) / 256; out[2] = (long long)tot; }
}

// G: row dot from shared memory, 16 warps, each `rows` rows of K=1024 fp16.  out[0] = cycles per row per warp
__device__ __forceinline__ float dot8(const uint4 w, const float *a, float acc) {
  const __half2 *h = reinterpret_cast<const __half2 *>(&w);
#pragma unroll
  for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); acc = fmaf(f.x, a[2 * i], acc); acc = fmaf(f.y, a[2 * i + 1], acc); }
  return acc;
}
__global__ void k_rowdot(long long *out, int rows) {
  extern __shared__ __align__(16) unsigned char ring[];
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  for (int i = threadIdx.x; i < 16 * 2048 / 4; i += blockDim.x) reinterpret_cast<unsigned *>(ring)[i] = 0x3c003c00u;
  __syncthreads();
  float a[32];
  for (int i = 0; i < 32; ++i) a[i] = 0.001f * (lane + i);
  float best = -1e30f;
  long long t0 = clock64();
  for (int r = 0; r < rows; ++r) {
    const uint4 *w = reinterpret_cast<const uint4 *>(ring + ((warp + r) & 15) * 2048);
    float acc[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) acc[j] = dot8(w[j * 32 + lane], &a[j * 8], 0.f);
    float v = (acc[0] + acc[1]) + (acc[2] + acc[3]);
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    if (v > best) best = v;
  }
  long long t1 = clock64();
  if (threadIdx.x == 0) { out[0] = (t1 - t0) / rows; out[1] = (long long)best; }
}

int main() {
  cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, 0));
  const int nsm = prop.multiProcessorCount;
  printf("device %s, %d SMs, clock %d kHz\n", prop.name, nsm, prop.clockRate);
  long long *out; CK(cudaMallocManaged(&out, 4096 * 8));
  int *err; CK(cudaMallocManaged(&err, 4)); *err = 0;
  // A
  k_timers<<<1, 1>>>(out); CK(cudaDeviceSynchronize());
  printf("A: clock64 %lld cycles/read, globaltimer %lld cycles/read\n", out[0], out[1]);
  // B, C
  {
    const int N = 8192; std::vector<unsigned long long> h(N);
    for (int i = 0; i < N; ++i) h[i] = (unsigned long long)((i * 1031 + 17) % N);
    unsigned long long *chain, *hot; int *stop;
    CK(cudaMalloc(&chain, N * 8)); CK(cudaMemcpy(chain, h.data(), N * 8, cudaMemcpyHostToDevice));
    CK(cudaMalloc(&hot, 4096 * 8)); CK(cudaMemset(hot, 0, 4096 * 8));
    CK(cudaMalloc(&stop, 4));
    for (int contend = 0; contend <= 1; ++contend) {
      CK(cudaMemset(stop, 0, 4));
      k_chase<<<contend ? nsm : 1, 512>>>(chain, 2000, hot, 1024, contend, stop, out); CK(cudaDeviceSynchronize());
      printf("%s: L2 relaxed.gpu load latency %lld cycles (%s)\n", contend ? "C" : "B", out[0], contend ? "147 CTAs x 512 threads polling 1024 words" : "idle GPU");
    }
  }
  // D
  {
    unsigned long long *words; CK(cudaMalloc(&words, 4096));
    int pairs[4][2] = {{0, 1}, {0, 2}, {0, nsm / 2}, {0, nsm - 1}};
    for (auto &pr : pairs) {
      CK(cudaMemset(words, 0, 4096)); out[3] = 0;
      k_pingpong<<<nsm, 32>>>(words, pr[0], pr[1], 2000, out); CK(cudaDeviceSynchronize());
      printf("D: ping-pong CTA %d <-> %d (SM %lld <-> %lld): %lld ns one-way, %lld cycles (err %lld)\n", pr[0], pr[1], out[2], out[4], out[0], out[1], out[3]);
    }
  }
  // E
  {
    unsigned long long *buf; CK(cudaMalloc(&buf, 2 * 4096 * 8));
    int nw[3] = {1024, 2048, 3072}; int sl[3] = {0, 50, 200};
    for (int n : nw) for (int s : sl) {
      CK(cudaMemset(buf, 0, 2 * 4096 * 8));
      int rounds = 200;
      void *args[] = {&buf, &n, &rounds, &s, &out, &err};
      CK(cudaLaunchCooperativeKernel((void *)k_exchange, dim3(nsm), dim3(512), args, 0, 0)); CK(cudaDeviceSynchronize());
      long long mx = 0, sum = 0; for (int i = 0; i < nsm; ++i) { sum += out[i]; if (out[i] > mx) mx = out[i]; }
      printf("E: LL all-to-all, %d words, sleep %d ns: %lld cycles/round mean (max %lld) err %d\n", n, s, sum / nsm, mx, *err);
    }
    float *data; unsigned *flags; CK(cudaMalloc(&data, 2 * 4096 * 4)); CK(cudaMalloc(&flags, 2 * 256 * 4));
    for (int n : nw) {
      CK(cudaMemset(flags, 0, 2 * 256 * 4));
      int rounds = 200;
      void *args[] = {&data, &flags, &n, &rounds, &out, &err};
      CK(cudaLaunchCooperativeKernel((void *)k_exchange_flags, dim3(nsm), dim3(512), args, 0, 0)); CK(cudaDeviceSynchronize());
      long long mx = 0, sum = 0; for (int i = 0; i < nsm; ++i) { sum += out[i]; if (out[i] > mx) mx = out[i]; }
      printf("E2: flag all-to-all, %d words: %lld cycles/round mean (max %lld) err %d\n", n, sum / nsm, mx, *err);
    }
  }
  // F
  k_barrier<<<1, 512>>>(out); CK(cudaDeviceSynchronize());
  printf("F: bar.sync(512) %lld cycles, block_sum (2 barriers) %lld cycles\n", out[0], out[1]);
  // G
  CK(cudaFuncSetAttribute(k_rowdot, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768));
  k_rowdot<<<1, 512, 32768>>>(out, 4096); CK(cudaDeviceSynchronize());
  printf("G: row dot K=1024 from smem, 16 warps: %lld cycles per row per warp\n", out[0]);
  k_rowdot<<<nsm, 512, 32768>>>(out, 4096); CK(cudaDeviceSynchronize());
  printf("G: same on all SMs: %lld cycles per row per warp\n", out[0]);
  return 0;
}
