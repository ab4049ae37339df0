// Probe: what scattered reductions and gathers cost on this GPU, next to plain streaming.
// Streams 1e7 (index, weight) pairs with 128-bit loads from a rotating 800 MB pool and, per pair,
//   red_f32 : red.global.add.f32 into a vector of `range` floats     (the CSR event scatter's access pattern)
//   stream  : nothing                                               (the HBM roofline of the same stream)
//   red_u32 : red.global.add.u32
//   gather  : one 4-byte load from the vector                        (the CSR gather's access pattern)
//   red_smem: atomicAdd(float) on a 32K-float shared-memory array
// Build and run:  nvcc -O3 -gencode arch=compute_100a,code=sm_100a -o l2_reduction_probe l2_reduction_probe.cu && ./l2_reduction_probe
// Needs ~1 GB of device memory and a few seconds.
#include <cstdio>
#include <cstdlib>
#include <vector>
#include <cuda_runtime.h>
#define CK(x) do{cudaError_t e=(x); if(e!=cudaSuccess){printf("err %s line %d\n", cudaGetErrorString(e), __LINE__); exit(1);} }while(0)

__global__ void k_red(const uint4* __restrict__ idx, const float4* __restrict__ w, float* y, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    uint4 c = idx[i]; float4 v = w[i];
    atomicAdd(y + c.x, v.x); atomicAdd(y + c.y, v.y); atomicAdd(y + c.z, v.z); atomicAdd(y + c.w, v.w);
  }
}
__global__ void k_red_u32(const uint4* __restrict__ idx, unsigned* y, size_t n4) {
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    uint4 c = idx[i];
    atomicAdd(y + c.x, 1u); atomicAdd(y + c.y, 1u); atomicAdd(y + c.z, 1u); atomicAdd(y + c.w, 1u);
  }
}
__global__ void k_stream(const uint4* __restrict__ idx, const float4* __restrict__ w, float* y, size_t n4) {
  float acc = 0; unsigned x = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    uint4 c = idx[i]; float4 v = w[i];
    x ^= c.x ^ c.y ^ c.z ^ c.w; acc += v.x + v.y + v.z + v.w;
  }
  if (acc == 1.2345f && x == 77) y[0] = acc;
}
__global__ void k_gather(const uint4* __restrict__ idx, const float4* __restrict__ w, const float* __restrict__ y, float* out, size_t n4) {
  float acc = 0;
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    uint4 c = idx[i]; float4 v = w[i];
    acc += v.x * __ldg(y + c.x) + v.y * __ldg(y + c.y) + v.z * __ldg(y + c.z) + v.w * __ldg(y + c.w);
  }
  if (acc == 1.2345f) out[0] = acc;
}
// red into shared memory (range-limited), to see smem atomic rate
__global__ void k_red_smem(const uint4* __restrict__ idx, const float4* __restrict__ w, float* y, size_t n4, unsigned mask) {
  extern __shared__ float s[];
  for (unsigned i = threadIdx.x; i <= mask; i += blockDim.x) s[i] = 0;
  __syncthreads();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n4; i += (size_t)gridDim.x * blockDim.x) {
    uint4 c = idx[i]; float4 v = w[i];
    atomicAdd(s + (c.x & mask), v.x); atomicAdd(s + (c.y & mask), v.y); atomicAdd(s + (c.z & mask), v.z); atomicAdd(s + (c.w & mask), v.w);
  }
  __syncthreads();
  if (threadIdx.x == 0 && s[0] == 1.2345f) y[0] = s[0];
}

int main() {
  const size_t N = 100000000;  // total elements (10 segments of 1e7)
  const size_t SEG = 10000000;
  std::vector<unsigned> h(N);
  unsigned s = 12345;
  unsigned *idx; float *w, *y; 
  CK(cudaMalloc(&idx, N * 4)); CK(cudaMalloc(&w, N * 4)); CK(cudaMalloc(&y, 64 << 20));
  CK(cudaMemset(w, 0, N * 4)); CK(cudaMemset(y, 0, 64 << 20));
  cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  int sms = 148;
  for (unsigned range : {1000000u, 125000u, 16000000u}) {
    for (size_t i = 0; i < N; ++i) { s = s * 1664525u + 1013904223u; h[i] = (unsigned)(((unsigned long long)(s >> 4) * range) >> 28); }
    CK(cudaMemcpy(idx, h.data(), N * 4, cudaMemcpyHostToDevice));
    for (int bps : {4, 8, 16}) for (int threads : {256, 512}) {
      if (bps * threads > 2048) continue;
      float best[5] = {1e9, 1e9, 1e9, 1e9, 1e9};
      for (int rep = 0; rep < 20; ++rep) {
        size_t off = (rep % 10) * SEG;
        const uint4* ip = (const uint4*)(idx + off); const float4* wp = (const float4*)(w + off);
        float ms;
        cudaEventRecord(e0); k_red<<<sms * bps, threads>>>(ip, wp, y, SEG / 4); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1); if (rep >= 2 && ms < best[0]) best[0] = ms;
        cudaEventRecord(e0); k_stream<<<sms * bps, threads>>>(ip, wp, y, SEG / 4); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1); if (rep >= 2 && ms < best[1]) best[1] = ms;
        cudaEventRecord(e0); k_red_u32<<<sms * bps, threads>>>(ip, (unsigned*)y, SEG / 4); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1); if (rep >= 2 && ms < best[2]) best[2] = ms;
        cudaEventRecord(e0); k_gather<<<sms * bps, threads>>>(ip, wp, y, y + (32 << 18), SEG / 4); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1); if (rep >= 2 && ms < best[3]) best[3] = ms;
        if (threads == 512 && bps == 4) { CK(cudaFuncSetAttribute(k_red_smem, cudaFuncAttributeMaxDynamicSharedMemorySize, 32768 * 4));
          cudaEventRecord(e0); k_red_smem<<<sms * 1, 1024, 32768 * 4>>>(ip, wp, y, SEG / 4, 32767u); cudaEventRecord(e1); CK(cudaEventSynchronize(e1)); cudaEventElapsedTime(&ms, e0, e1); if (rep >= 2 && ms < best[4]) best[4] = ms; }
      }
      printf("range %u bps %d thr %d : red_f32 %.2f us (%.1f G/s)  stream %.2f us (%.0f GB/s)  red_u32 %.2f us  gather %.2f us  red_smem %.2f us\n",
             range, bps, threads, best[0] * 1e3, 1e7 / best[0] * 1e-6, best[1] * 1e3, 8e7 / best[1] * 1e-6, best[2] * 1e3, best[3] * 1e3, best[4] * 1e3);
      fflush(stdout);
    }
  }
  return 0;
}
