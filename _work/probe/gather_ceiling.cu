// Random-gather throughput of the GPU (G gathers/s) for the access patterns an SpMV makes into x: uniformly random
// over vectors of several sizes, and local (+-w of a moving centre), for 2-byte and 8-byte elements.  16 independent
// gathers per thread, indices streamed with coalesced loads.  Gives the ceiling that bounds irregular SpMV.
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
template <typename V, int IPT>
__global__ void __launch_bounds__(256) gk(const int* __restrict__ idx, const V* __restrict__ x, float* out, long n) {
  long base = (long)blockIdx.x * 256 * IPT;
  int c[IPT];
  #pragma unroll
  for (int j=0;j<IPT;++j) { long i = base + threadIdx.x + j*256; c[j] = i < n ? __ldg(idx+i) : 0; }
  float acc = 0;
  #pragma unroll
  for (int j=0;j<IPT;++j) acc += (float)__ldg(x + c[j]);
  if (acc == 123456.789f) out[0] = acc;
}
// SpMV without the row logic: streams (index, value), gathers x, multiplies, reduces per thread.
template <typename V, int IPT>
__global__ void __launch_bounds__(128) gkv(const int* __restrict__ idx, const V* __restrict__ val, const V* __restrict__ x, float* out, long n) {
  long base = (long)blockIdx.x * 128 * IPT;
  int c[IPT]; V v[IPT];
  #pragma unroll
  for (int j=0;j<IPT;++j) { long i = base + threadIdx.x + j*128; c[j] = i < n ? __ldcs(idx+i) : 0; v[j] = i < n ? __ldcs(val+i) : V(0); }
  float acc = 0;
  #pragma unroll
  for (int j=0;j<IPT;++j) acc += (float)v[j] * (float)__ldg(x + c[j]);
  if (acc == 123456.789f) out[0] = acc;
}
// share p_uniform of the indices uniform over x (or over `hot` scattered columns when hot > 0), the rest within +-win
template <typename V> void run_mix(const char* name, long nx, long n, double p_uniform, int win, long hot, double p_hot) {
  std::vector<int> h(n);
  uint64_t s = 88172645463325252ull;
  for (long i=0;i<n;++i) { s ^= s<<13; s ^= s>>7; s ^= s<<17;
    double u = (double)(s >> 11) / 9007199254740992.0; uint64_t r = s * 0x9E3779B97F4A7C15ull >> 20;
    long c;
    if (u < p_uniform) c = r % nx;
    else if (u < p_uniform + p_hot) c = (long)((r % hot) * (double)nx / hot);
    else { long center = (long)((double)i / n * nx); c = center - win + (long)(r % (2*win+1)); if (c<0) c=0; if (c>=nx) c=nx-1; }
    h[i] = (int)c; }
  int* d; V* x; V* v; float* o; cudaMalloc(&d, n*4); cudaMalloc(&v, n*sizeof(V)); cudaMalloc(&x, nx*sizeof(V)); cudaMalloc(&o, 4);
  cudaMemcpy(d, h.data(), n*4, cudaMemcpyHostToDevice); cudaMemset(x, 0, nx*sizeof(V)); cudaMemset(v, 0, n*sizeof(V));
  const int IPT=16; int grid = (n + 128*IPT - 1)/(128*IPT);
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  for (int i=0;i<3;++i) gkv<V,IPT><<<grid,128>>>(d,v,x,o,n);
  cudaEventRecord(e0); for (int i=0;i<20;++i) gkv<V,IPT><<<grid,128>>>(d,v,x,o,n); cudaEventRecord(e1); cudaEventSynchronize(e1);
  float ms; cudaEventElapsedTime(&ms,e0,e1); ms/=20;
  printf("%-28s x=%7.1f MB elem=%zuB n=%ldM : %.3f ms  %.1f Gnnz/s  (stream %.0f GB/s)\n", name, nx*sizeof(V)/1e6, sizeof(V), n/1000000, ms, n/ms/1e6, n*(4+sizeof(V))/ms/1e6);
  cudaFree(d); cudaFree(v); cudaFree(x); cudaFree(o);
}
template <typename V> void run(const char* name, long nx, long n, int mode, int win) {
  std::vector<int> h(n);
  uint64_t s = 88172645463325252ull;
  for (long i=0;i<n;++i) { s ^= s<<13; s ^= s>>7; s ^= s<<17;
    long c;
    if (mode==0) c = s % nx;                                  // uniform
    else { long center = (long)((double)i / n * nx); c = center - win + (long)(s % (2*win+1)); if (c<0) c=0; if (c>=nx) c=nx-1; }  // local
    h[i] = (int)c; }
  int* d; V* x; float* o; cudaMalloc(&d, n*4); cudaMalloc(&x, nx*sizeof(V)); cudaMalloc(&o, 4);
  cudaMemcpy(d, h.data(), n*4, cudaMemcpyHostToDevice); cudaMemset(x, 0, nx*sizeof(V));
  const int IPT=16; int grid = (n + 256*IPT - 1)/(256*IPT);
  cudaEvent_t e0,e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
  for (int i=0;i<3;++i) gk<V,IPT><<<grid,256>>>(d,x,o,n);
  cudaEventRecord(e0); for (int i=0;i<20;++i) gk<V,IPT><<<grid,256>>>(d,x,o,n); cudaEventRecord(e1); cudaEventSynchronize(e1);
  float ms; cudaEventElapsedTime(&ms,e0,e1); ms/=20;
  printf("%-28s x=%7.1f MB elem=%zuB n=%ldM : %.3f ms  %.1f Ggather/s  (idx stream %.0f GB/s)\n", name, nx*sizeof(V)/1e6, sizeof(V), n/1000000, ms, n/ms/1e6, n*4/ms/1e6);
  cudaFree(d); cudaFree(x); cudaFree(o);
}
int main() {
  long n = 64L<<20;
  run<__half>("uniform half", 2L<<20, n, 0, 0);
  run<__half>("uniform half", 32L<<20, n, 0, 0);
  run<__half>("uniform half", 256L<<20, n, 0, 0);
  run<double>("uniform double", 1572864, n, 0, 0);
  run<double>("uniform double", 8L<<20, n, 0, 0);
  run<double>("uniform double", 64L<<20, n, 0, 0);
  run<__half>("local+-256 half", 2L<<20, n, 1, 256);
  run<__half>("local+-4096 half", 2L<<20, n, 1, 4096);
  run<double>("local+-256 double", 8L<<20, n, 1, 256);
  run<double>("local+-4096 double", 8L<<20, n, 1, 4096);
  // index + value streams with the column mixes of the benchmark shapes (no row logic: an upper bound for a CSR kernel)
  run_mix<__half>("mix 40%uni 60%+-256 half", 2000000, n, 0.4, 256, 0, 0.0);
  run_mix<__half>("mix 60%uni 40%hot80k half", 4000000, n, 0.6, 256, 80000, 0.4);
  run_mix<double>("mix 50%uni 50%+-1024 f64", 64000000, n, 0.5, 1024, 0, 0.0);
  run_mix<double>("band +-4096 f64", 1572864, n, 0.0, 4096, 0, 0.0);
  return 0;
}
