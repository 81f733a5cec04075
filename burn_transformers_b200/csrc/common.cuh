// Shared helpers of the sm_100a kernels: element types, reductions, error reporting.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>

namespace bt {

enum DType : int { kF32 = 0, kBF16 = 1 };

// Last error text of the calling thread, read by bt_last_error().
char* error_buffer();
int fail(const char* fmt, ...);
// Kernel launches issued through this library since it was loaded (launches recorded into a CUDA
// graph count once, at capture).
void count_launch();

#define BT_CHECK(cond, ...)                                   \
  do {                                                        \
    if (!(cond)) return ::bt::fail(__VA_ARGS__);              \
  } while (0)

#define BT_LAUNCH_OK(name)                                                                   \
  do {                                                                                       \
    cudaError_t e_ = cudaGetLastError();                                                     \
    if (e_ != cudaSuccess) return ::bt::fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    ::bt::count_launch();                                                                    \
  } while (0)

// Programmatic dependent launch.  A kernel launched through launch_pdl may start while the kernel before it
// in the stream is still running; it must call pdl_wait() before it reads or writes anything that kernel
// touches (after the call the whole earlier grid has finished and its writes are visible).  What comes
// before pdl_wait() may only read memory that no kernel of the step writes: weights.  pdl_trigger() lets
// the next kernel of the stream begin its own prologue.  Both are no-ops in a kernel launched the plain way.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// BT_NO_PDL=1 in the environment launches every kernel fully serialised (for measurements).
bool pdl_enabled();

// Streaming multiprocessors of the current device (looked up once per device); 0 if it cannot be read.
int sm_count();

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                              int cluster_x, Args... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  int n = 0;
  attr[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[n].val.programmaticStreamSerializationAllowed = pdl_enabled() ? 1 : 0;
  ++n;
  if (cluster_x > 1) {
    attr[n].id = cudaLaunchAttributeClusterDimension;
    attr[n].val.clusterDim.x = cluster_x;
    attr[n].val.clusterDim.y = 1;
    attr[n].val.clusterDim.z = 1;
    ++n;
  }
  cfg.attrs = attr;
  cfg.numAttrs = n;
  return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define BT_PDL_OK(name, call)                                                                 \
  do {                                                                                        \
    cudaError_t e_ = (call);                                                                  \
    if (e_ != cudaSuccess) return ::bt::fail("%s: launch failed: %s", name, cudaGetErrorString(e_)); \
    ::bt::count_launch();                                                                     \
  } while (0)

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
  return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < nwarp ? scratch[lane] : 0.f;
    w = warp_sum(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int nwarp = (blockDim.x + 31) >> 5;
  v = warp_max(v);
  __syncthreads();
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float w = lane < nwarp ? scratch[lane] : -INFINITY;
    w = warp_max(w);
    if (lane == 0) scratch[32] = w;
  }
  __syncthreads();
  return scratch[32];
}

// tanh-form GELU ("gelu_new") and erf-form GELU, full-precision library functions.
__device__ __forceinline__ float gelu_tanh(float x) {
  const float k = 0.7978845608028654f;  // sqrt(2/pi)
  return 0.5f * x * (1.f + tanhf(k * (x + 0.044715f * x * x * x)));
}
__device__ __forceinline__ float gelu_erf(float x) {
  return 0.5f * x * (1.f + erff(x * 0.7071067811865476f));
}

enum Activation : int { kActNone = 0, kActGeluTanh = 1, kActGeluErf = 2 };

__device__ __forceinline__ float apply_activation(float v, int act) {
  if (act == kActGeluTanh) return gelu_tanh(v);
  if (act == kActGeluErf) return gelu_erf(v);
  return v;
}

// Where the keys and values of one attention call live.
//  paged: pool[page][kv_head][page_size][head_dim], page = table[seq * table_stride + (pos / page_size) % table_len]
//  packed: the step's own projections, rows of `row_stride` elements, row = seq_start[seq] + pos
struct KvView {
  const void* k;
  const void* v;
  const int* table;      // null => packed
  int table_stride;
  int table_len;         // pages a sequence cycles through (ring) or may hold (full)
  int page_size;
  long long row_stride;  // packed: elements between consecutive tokens
  const int* seq_start;  // packed: first row of each sequence
};

template <typename T>
__device__ __forceinline__ const T* kv_row(const void* base, const KvView& kv, int seq, int kv_head, int n_kv_heads,
                                           int head_dim, int pos) {
  const T* b = reinterpret_cast<const T*>(base);
  if (kv.table) {
    const int lp = pos / kv.page_size;
    const int page = kv.table[(long long)seq * kv.table_stride + (lp % kv.table_len)];
    return b + (((long long)page * n_kv_heads + kv_head) * kv.page_size + (pos - lp * kv.page_size)) * head_dim;
  }
  return b + ((long long)kv.seq_start[seq] + pos) * kv.row_stride + (long long)kv_head * head_dim;
}

}  // namespace bt
