// An int8 InnerProduct entry point for callers that must not allocate.
//
// Some hosts of this library run where device allocation is off the table: a
// real-time loop that was given its buffers at start-up and may not touch the
// allocator again, a plug-in sandbox whose policy forbids cudaMalloc, or a
// process that has already handed every byte of the GPU to its own pool.  The
// regular path (ncnn_b200_load + run) allocates an arena and staging buffers, so
// it is closed to them.  This file offers one operator they can still call: the
// quantised InnerProduct.  The operator needs one piece of scratch -- the int8
// copy of the fp32 activations -- and takes it from a fixed array that lives in
// the library image itself, so no allocation call of any kind is made here.
//
// Consequences of the fixed array, all of which the caller must know:
//  * every GPU on which the library's code gets loaded carries kNoAllocScratchBytes (8 MiB) from
//    that moment until the process exits (the CUDA runtime loads the module lazily, typically at
//    the first call into the library on that device; make that call at start-up);
//  * M*K may not exceed that size; larger requests are refused, never truncated;
//  * all calls on one device share the array, and it keeps whatever the last call
//    left there (nothing in it needs clearing: each call overwrites the M*K bytes
//    it reads back), so two calls that overlap on the GPU -- different streams,
//    or different host threads -- race and must be serialised by the caller;
//  * the first call on a device looks up the array's device address
//    (cudaGetSymbolAddress), so make that first call before starting any stream
//    capture;
//  * the looked-up address is cached per device for the life of the process: a host program that
//    calls cudaDeviceReset() must not use this entry point on that device afterwards;
//  * `weight` may sit at any byte address (a sub-allocated blob, say): rows are read four bytes
//    at a time only when the pointer and K allow it, byte by byte otherwise.
#include "../../include/ncnn_b200.h"

#include <mutex>
#include <string>

#include <cuda_runtime.h>

#include "tc_gemm.cuh"

namespace nb {
void set_global_error(const std::string& message);  // c_api.cu
}

namespace {

constexpr size_t kNoAllocScratchBytes = 8u << 20;
constexpr int kMaxDevices = 64;

// The name below is only a host-side handle; the device address is fetched per device.
static __device__ __align__(256) unsigned char g_no_alloc_scratch[kNoAllocScratchBytes];

std::mutex g_setup_mutex;
void* g_scratch_address[kMaxDevices] = {};

__global__ void k_na_quantize(const float* __restrict__ x, int8_t* __restrict__ xq, long long count,
                              float scale) {
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < count;
       i += static_cast<long long>(gridDim.x) * blockDim.x)
    xq[i] = static_cast<int8_t>(nb::quantize_rha(x[i], scale));
}

// y[m][n] = act(float(sum_k xq[m][k]*w[n][k]) * 1/(s_w[n]*s_in) + bias[n]); one thread per output.
__global__ void k_na_inner_product(const int8_t* __restrict__ xq, const int8_t* __restrict__ w,
                                   const float* __restrict__ weight_scales, float input_scale,
                                   const float* __restrict__ bias, float* __restrict__ y, long long M,
                                   int K, int N, int relu, int words) {
  const long long total = M * N;
  for (long long i = blockIdx.x * static_cast<long long>(blockDim.x) + threadIdx.x; i < total;
       i += static_cast<long long>(gridDim.x) * blockDim.x) {
    const int n = static_cast<int>(i % N);
    const long long m = i / N;
    const int8_t* a = xq + m * K;
    const int8_t* b = w + static_cast<long long>(n) * K;
    int acc = 0;
    int k = 0;
    if (words) {  // both operands 4-byte aligned in every row (checked on the host)
      for (; k < K; k += 4)
        acc = __dp4a(*reinterpret_cast<const int*>(a + k), *reinterpret_cast<const int*>(b + k), acc);
    }
    for (; k < K; ++k) acc += static_cast<int>(a[k]) * static_cast<int>(b[k]);
    const float ws = weight_scales[n];
    const float r = ws == 0.0f ? 0.0f : __fdiv_rn(1.0f, __fmul_rn(ws, input_scale));
    float v = __fmul_rn(static_cast<float>(acc), r);
    if (bias != nullptr) v = __fadd_rn(v, bias[n]);
    if (relu) v = fmaxf(v, 0.0f);
    y[i] = v;
  }
}

int fail(int status, const std::string& message) {
  nb::set_global_error(message);
  return status;
}

}  // namespace

extern "C" int ncnn_b200_inner_product_int8_noalloc(const float* x, const int8_t* weight,
                                                    const float* weight_scales, float input_scale,
                                                    const float* bias, float* y, int64_t m, int32_t k,
                                                    int32_t n, int32_t relu, void* stream) {
  if (x == nullptr || weight == nullptr || weight_scales == nullptr || y == nullptr)
    return fail(NCNN_B200_STATUS_NULL_POINTER, "inner_product_int8_noalloc: NULL argument");
  if (m <= 0 || k <= 0 || n <= 0 || !(input_scale > 0.0f))
    return fail(NCNN_B200_STATUS_INVALID_SHAPE,
                "inner_product_int8_noalloc: m, k, n and input_scale must be positive");
  // (a quotient, not a product: m*k could wrap for absurd m)
  if (m > static_cast<int64_t>(kNoAllocScratchBytes / static_cast<uint64_t>(k)))
    return fail(NCNN_B200_STATUS_OUTPUT_CAPACITY,
                "inner_product_int8_noalloc: m = " + std::to_string(m) + " rows of k = " + std::to_string(k) +
                    " int8 activations exceed the built-in scratch of " +
                    std::to_string(kNoAllocScratchBytes) + " bytes; split the rows into several calls");
  int device = 0;
  if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices)
    return fail(NCNN_B200_STATUS_RUNTIME, "inner_product_int8_noalloc: no usable current CUDA device");
  void* scratch = nullptr;
  {
    // once per device, with that device current: translate the symbol into a device address
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (g_scratch_address[device] == nullptr) {
      void* address = nullptr;
      const cudaError_t e = cudaGetSymbolAddress(&address, g_no_alloc_scratch);
      if (e != cudaSuccess || address == nullptr)
        return fail(NCNN_B200_STATUS_RUNTIME,
                    std::string("inner_product_int8_noalloc: cudaGetSymbolAddress failed: ") +
                        cudaGetErrorString(e));
      g_scratch_address[device] = address;
    }
    scratch = g_scratch_address[device];
  }
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int8_t* xq = static_cast<int8_t*>(scratch);
  const long long count = static_cast<long long>(m) * k;
  const int grid_q = static_cast<int>(std::min<long long>((count + 255) / 256, 148 * 16));
  k_na_quantize<<<grid_q, 256, 0, st>>>(x, xq, count, input_scale);
  const long long outputs = static_cast<long long>(m) * n;
  const int grid_m = static_cast<int>(std::min<long long>((outputs + 255) / 256, 148 * 16));
  // the scratch rows start at multiples of k from a 256-byte boundary; the caller's weight may not
  const int words = (k % 4 == 0 && (reinterpret_cast<uintptr_t>(weight) & 3u) == 0) ? 1 : 0;
  k_na_inner_product<<<grid_m, 256, 0, st>>>(xq, weight, weight_scales, input_scale, bias, y, m, k, n,
                                             relu ? 1 : 0, words);
  const cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess)
    return fail(NCNN_B200_STATUS_RUNTIME,
                std::string("inner_product_int8_noalloc: launch failed: ") + cudaGetErrorString(e));
  return NCNN_B200_STATUS_SUCCESS;
}
