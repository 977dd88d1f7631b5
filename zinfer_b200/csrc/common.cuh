// Shared helpers of the sm_100a kernels: dtype tags, loads that widen to 32-bit,
// reductions with a fixed order, and the error channel of the C entry points.
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define ZI_F32 0
#define ZI_BF16 1

// Entry points return 0, a cudaError_t (> 0), or ZI_REFUSED (< 0) with the reason
// in zi_last_error().
#define ZI_REFUSED (-1)

extern "C" const char* zi_last_error();
int zi_refuse(const char* fmt, ...);
int zi_check_launch(const char* what);

template <typename T> struct DTypeTag;
template <> struct DTypeTag<float> { static constexpr int value = ZI_F32; };
template <> struct DTypeTag<__nv_bfloat16> { static constexpr int value = ZI_BF16; };

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

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

// The arithmetic of the per-head norm and the rotation, with every rounding spelled out, so that
// the kernels that make keys (alone, or fused into the decode attention) store the same bits
// whatever the compiler would contract.
__device__ __forceinline__ float sum_squares_step(float ss, float a, float b) { return __fmaf_rn(b, b, __fmaf_rn(a, a, ss)); }
__device__ __forceinline__ float norm_scale(float v, float w, float inv) { return __fmul_rn(__fmul_rn(v, w), inv); }
__device__ __forceinline__ void rotate_pair(float& x, float& y, float c, float s) {
  const float rx = __fsub_rn(__fmul_rn(x, c), __fmul_rn(y, s));
  const float ry = __fadd_rn(__fmul_rn(y, c), __fmul_rn(x, s));
  x = rx;
  y = ry;
}

// Sum over a block of up to 1024 threads; every thread receives the result.  The
// order of additions depends only on blockDim, never on the data's place in a batch.
__device__ __forceinline__ float block_sum(float v, float* scratch /* >= 33 floats */) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarp = (blockDim.x + 31) >> 5;
  v = warp_sum(v);
  __syncthreads();  // scratch may still be read from an earlier call
  if (lane == 0) scratch[warp] = v;
  __syncthreads();
  if (warp == 0) {
    float t = lane < nwarp ? scratch[lane] : 0.f;
    t = warp_sum(t);
    if (lane == 0) scratch[32] = t;
  }
  __syncthreads();
  return scratch[32];
}

// --------------------------------------------------- programmatic dependent launch
// Every kernel is launched with programmatic stream serialization (unless switched off):
// the next kernel of the stream may start its prologue while this one drains.  A kernel
// therefore calls pdl_wait() before it reads anything an earlier kernel wrote (and every
// kernel calls it once, so that completion stays transitive along the stream), and
// pdl_launch_dependents() as soon as the next kernel may begin to start.
//
// Built with -DZI_TRACE (ZINFER_B200_TRACE=1 when the library is built), both calls also leave a time
// stamp: thread 0 of a kernel's first block records %globaltimer when the kernel starts (stamp 0) and
// when the kernels before it have completed (stamp 1) into a buffer given by zi_trace_set_<file>().
// From these a step's timeline can be read as it runs inside the chain, overlaps included, which
// no profiler that serialises kernels shows.  Without the flag none of this is compiled.
#ifdef ZI_TRACE
constexpr unsigned ZI_TRACE_CAPACITY = 8192;
static __device__ unsigned long long* zi_trace_ptr = nullptr;   // word 0: number of stamps; then the stamps
__device__ __forceinline__ void zi_stamp(unsigned what) {
  unsigned long long* t = zi_trace_ptr;
  if (t && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0 && threadIdx.x == 0) {
    unsigned long long now;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(now));
    const unsigned idx = atomicAdd((unsigned*)t, 1u);
    if (idx < ZI_TRACE_CAPACITY) t[1 + idx] = (now << 2) | what;
  }
}
// one setter per source file (each has its own copy of the pointer)
#define ZI_TRACE_SETTER(file) \
  extern "C" int zi_trace_set_##file(void* p) { return (int)cudaMemcpyToSymbol(zi_trace_ptr, &p, sizeof(p)); }
#else
__device__ __forceinline__ void zi_stamp(unsigned) {}
#define ZI_TRACE_SETTER(file)
#endif
__device__ __forceinline__ void pdl_wait() {
  asm volatile("griddepcontrol.wait;" ::: "memory");
  zi_stamp(1);
}
__device__ __forceinline__ void pdl_launch_dependents() {
  zi_stamp(0);
  asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

extern int g_zi_pdl_enabled;

template <typename... KArgs, typename... Args>
inline cudaError_t zi_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                             Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = g_zi_pdl_enabled ? 1 : 0;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

#define ZI_DISPATCH_DTYPE(dtype, T, ...)                                   \
  do {                                                                     \
    if ((dtype) == ZI_F32) { using T = float; __VA_ARGS__; }               \
    else if ((dtype) == ZI_BF16) { using T = __nv_bfloat16; __VA_ARGS__; } \
    else return zi_refuse("unknown dtype tag %d", (int)(dtype));           \
  } while (0)
