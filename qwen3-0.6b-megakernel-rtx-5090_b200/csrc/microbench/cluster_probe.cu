// Stand-alone microbenchmark of thread-block-cluster primitives on sm_100a, for a decode kernel that would keep
// the attention + O-proj and the MLP halves of a layer inside one 16-CTA cluster:
//   (1) can 8 clusters of 16 CTAs with ~200 KB of dynamic shared memory and 416 threads each be co-resident;
//   (2) one all-to-all round inside a cluster through distributed shared memory: every CTA pushes `nvals` tagged
//       8-byte words to every peer (st.shared::cluster) and waits, bounded, until all peers' words arrived;
//   (3) the hardware cluster barrier (barrier.cluster.arrive + wait) for comparison.
// Every spin is bounded.  Build and run:
//   nvcc -O3 -std=c++17 -gencode arch=compute_100a,code=sm_100a -o cluster_probe cluster_probe.cu && ./cluster_probe
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("CUDA error %s at line %d\n", cudaGetErrorString(e), __LINE__); return 1; } } while (0)

__device__ __forceinline__ uint32_t s32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ uint32_t cluster_rank() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r)); return r; }
__device__ __forceinline__ uint32_t cluster_size() { uint32_t r; asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(r)); return r; }
// address of `local` (a shared::cta address) in CTA `rank` of the cluster
__device__ __forceinline__ uint32_t map_to(uint32_t local, uint32_t rank) {
  uint32_t r; asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank)); return r;
}
__device__ __forceinline__ void st_cluster_u64(uint32_t addr, unsigned long long v) {
  asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(addr), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_local_u64(const volatile unsigned long long *p) { return *p; }
__device__ __forceinline__ void cluster_barrier() {
  asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
  asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

// mode 0: DSMEM all-to-all of nvals words per CTA; mode 1: hardware cluster barrier only
__global__ void k_probe(int nvals, int rounds, int mode, long long *out, int *err) {
  extern __shared__ __align__(16) unsigned char smem[];
  // inbox[src_rank][nvals] of tagged words, at the start of dynamic shared memory (same offset in every CTA)
  volatile unsigned long long *inbox = reinterpret_cast<volatile unsigned long long *>(smem);
  const uint32_t me = cluster_rank(), n = cluster_size();
  const int tid = threadIdx.x, nthr = blockDim.x;
  for (int i = tid; i < (int)n * nvals; i += nthr) inbox[i] = 0ull;
  cluster_barrier();   // every inbox is zeroed before anybody pushes
  long long t0 = clock64();
  for (int r = 1; r <= rounds; ++r) {
    if (mode == 0) {
      // push: thread t handles (peer, value) pairs
      for (int i = tid; i < (int)n * nvals; i += nthr) {
        const uint32_t peer = i / nvals, v = i % nvals;
        const uint32_t local = s32(const_cast<unsigned long long *>(inbox) + me * nvals + v);
        st_cluster_u64(map_to(local, peer), ((unsigned long long)r << 32) | (me * 1000u + v));
      }
      // wait for everybody's words (bounded)
      for (int i = tid; i < (int)n * nvals; i += nthr) {
        // a fast peer may already have pushed a later round: tags only grow, so wait for "at least r"
        long long spins = 0;
        while ((uint32_t)(ld_local_u64(inbox + i) >> 32) < (uint32_t)r) {
          if (++spins > 200000) { *err = 1; break; }
        }
        if ((uint32_t)ld_local_u64(inbox + i) != (uint32_t)((i / nvals) * 1000u + (i % nvals)) && !*err) *err = 2;
      }
      __syncthreads();
    } else {
      cluster_barrier();
    }
  }
  long long dt = clock64() - t0;
  cluster_barrier();   // nobody exits while a peer may still push into its shared memory
  if (tid == 0) out[blockIdx.x] = dt / rounds;
}

int main() {
  setvbuf(stdout, nullptr, _IONBF, 0);
  cudaDeviceProp prop; CK(cudaGetDeviceProperties(&prop, 0));
  printf("%s, %d SMs\n", prop.name, prop.multiProcessorCount);
  long long *out; CK(cudaMallocManaged(&out, 1024 * 8));
  int *err; CK(cudaMallocManaged(&err, 4));
  const int threads = 416;
  CK(cudaFuncSetAttribute(k_probe, cudaFuncAttributeNonPortableClusterSizeAllowed, 1));
  const size_t smem_big = 200 * 1024;
  CK(cudaFuncSetAttribute(k_probe, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem_big));
  int csizes[3] = {4, 8, 16};
  for (int cs : csizes) {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cs; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.blockDim = dim3(threads); cfg.dynamicSmemBytes = smem_big; cfg.attrs = attr; cfg.numAttrs = 1;
    int max_clusters = 0;
    cfg.gridDim = dim3(cs);   // the query wants a valid grid
    cudaError_t qe = cudaOccupancyMaxActiveClusters(&max_clusters, k_probe, &cfg);
    printf("cluster size %2d, %zu KB smem, %d threads: max co-resident clusters %d (%s) -> %d CTAs\n", cs, smem_big / 1024,
           threads, max_clusters, cudaGetErrorString(qe), max_clusters * cs);
    if (qe != cudaSuccess || max_clusters < 1) { cudaGetLastError(); continue; }
    const int nclusters = max_clusters < 148 / cs ? max_clusters : 148 / cs;
    cfg.gridDim = dim3(nclusters * cs);
    int nvals_list[4] = {32, 64, 260, 1024 / 16 * 16};
    for (int mode = 0; mode < 2; ++mode)
      for (int nv : nvals_list) {
        if (mode == 1 && nv != 32) continue;
        if ((size_t)cs * nv * 8 > smem_big) continue;
        *err = 0;
        CK(cudaLaunchKernelEx(&cfg, k_probe, nv, 200, mode, out, err));
        CK(cudaDeviceSynchronize());
        long long mx = 0, mn = 1ll << 60;
        for (int i = 0; i < nclusters * cs; ++i) { if (out[i] > mx) mx = out[i]; if (out[i] < mn) mn = out[i]; }
        if (mode == 0)
          printf("  %d clusters x %d: DSMEM all-to-all, %4d words per CTA -> every peer: %lld .. %lld cycles per round (err %d)\n",
                 nclusters, cs, nv, mn, mx, *err);
        else
          printf("  %d clusters x %d: barrier.cluster arrive+wait: %lld .. %lld cycles per round\n", nclusters, cs, mn, mx);
      }
  }
  return 0;
}
