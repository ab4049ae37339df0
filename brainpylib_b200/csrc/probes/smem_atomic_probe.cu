// Probe: shared-memory atomic throughput per SM for float, 32-bit and 64-bit integer adds at random
// addresses (plus a racy plain read-modify-write as an upper bound), for 1 or 2 CTAs per SM.
// Build and run:  nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o smem_atomic_probe smem_atomic_probe.cu && ./smem_atomic_probe
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); exit(1);} }while(0)

template<int MODE>
__global__ void k(unsigned* out, int iters, unsigned mask) {
  extern __shared__ unsigned long long s64[];
  float* sf = (float*)s64; unsigned* su = (unsigned*)s64;
  for (unsigned i = threadIdx.x; i <= mask; i += blockDim.x) s64[i] = 0;
  __syncthreads();
  unsigned x = threadIdx.x * 2654435761u + blockIdx.x * 40503u + 12345u;
  for (int it = 0; it < iters; ++it) {
    x = x * 1664525u + 1013904223u;
    unsigned a = (x >> 8) & mask;
    if (MODE == 0) atomicAdd(sf + a, 1.0f);
    else if (MODE == 1) atomicAdd(su + a, 1u);
    else if (MODE == 2) atomicAdd(s64 + a, 1ull);
    else if (MODE == 3) { sf[a] += 1.0f; }   // non-atomic RMW (racy) as an upper bound
    else if (MODE == 4) asm volatile("red.shared.add.f32 [%0], %1;" :: "r"((unsigned)__cvta_generic_to_shared(sf + a)), "f"(1.0f) : "memory");
  }
  __syncthreads();
  if (threadIdx.x == 0) out[blockIdx.x] = su[0];
}

int main() {
  unsigned* out; CK(cudaMalloc(&out, 4096 * 4));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  const int iters = 2000;
  const char* names[] = {"atomicAdd f32", "atomicAdd u32", "atomicAdd u64", "plain rmw f32", "red.shared f32"};
  for (int mode = 0; mode < 5; ++mode) for (int threads : {256, 512, 1024}) for (int bps : {1, 2}) {
    if (threads * bps > 2048) continue;
    size_t smem = 16384 * 8;  // 16K 8-byte slots = 128 KB ... too big for 2 blocks; use mask accordingly
    unsigned mask = 16383;
    if (bps == 2) { smem = 8192 * 8; mask = 8191; }
    void (*fn)(unsigned*, int, unsigned) = mode == 0 ? k<0> : mode == 1 ? k<1> : mode == 2 ? k<2> : mode == 3 ? k<3> : k<4>;
    CK(cudaFuncSetAttribute(fn, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    float best = 1e9;
    for (int rep = 0; rep < 5; ++rep) {
      cudaEventRecord(e0); fn<<<148 * bps, threads, smem>>>(out, iters, mask); cudaEventRecord(e1); CK(cudaEventSynchronize(e1));
      float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
    }
    double total = 148.0 * bps * threads * iters;
    printf("%-16s thr %4d bps %d : %.1f us  %.0f G/s total  %.2f per clk per SM (1.965GHz)\n", names[mode], threads, bps, best * 1e3, total / best * 1e-6, total / best * 1e-6 / 148 / 1.965);
  }
  return 0;
}
