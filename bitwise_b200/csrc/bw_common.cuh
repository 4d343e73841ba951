// Shared declarations of the kernel libraries: error reporting, the exported-symbol macro,
// and the arithmetic that must give the same bits on the host and on the device.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#define BW_API extern "C" __attribute__((visibility("default")))

// Every exported function returns 0 on success. A non-zero value is either a CUDA error
// code (> 0) or an argument error (< 0); bw_last_error() gives the text of the latter.
namespace bw {

void set_error(const char* fmt, ...);

inline int launch_status() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) set_error("CUDA launch failed: %s", cudaGetErrorString(e));
  return static_cast<int>(e);
}

// Programmatic dependent launch: every kernel of the serving path is launched with the
// attribute below. pdl_launch() at its very start lets the NEXT kernel's blocks be placed on
// the SMs as soon as all of this kernel's blocks have started; pdl_wait() returns once the
// kernel before this one in the stream has completed and its writes are visible (and that
// kernel had itself waited for its predecessor, so everything earlier is complete too). Launch
// latency and block scheduling thus overlap the running kernels instead of following them. Before pdl_wait() a kernel reads only what no
// kernel of the same step writes: weights, the step's index arrays (copied to the device
// before the step's first kernel) and cache entries that earlier steps stored.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// What most kernels begin with. A launch of few blocks (a decode step's kernels) lets its
// successor be placed at once and then waits; a launch of many blocks waits first, so that the
// successor's blocks do not take SMs while this kernel still has blocks to place (measured:
// early placement speeds a decode step up by 4 % and slows a 2,048-token prefill down by 4 %).
__device__ __forceinline__ void pdl_enter() {
  const bool few = gridDim.x * gridDim.y * gridDim.z <= 296;
  if (few) pdl_launch();
  pdl_wait();
  if (!few) pdl_launch();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
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
  cfg.numAttrs = 1;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The same for a kernel whose blocks form clusters of two along x.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pdl_cluster2(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                       cudaStream_t stream, Args&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = stream;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  attr[1].id = cudaLaunchAttributeClusterDimension;
  attr[1].val.clusterDim.x = 2;
  attr[1].val.clusterDim.y = 1;
  attr[1].val.clusterDim.z = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// The first address at or after `raw` (the block's dynamic shared memory) that is a multiple of
// 1,024, found by pointer arithmetic. A pointer that went through an integer on its way is no
// longer known to point into shared memory, and every access through it becomes a generic load
// or store, which costs a chain of dependent reads twice the cycles.
__device__ __forceinline__ unsigned char* smem_align_1024(unsigned char* raw) {
  return raw + ((1024u - (static_cast<uint32_t>(__cvta_generic_to_shared(raw)) & 1023u)) & 1023u);
}

// ---- bounded waits and the failure word --------------------------------------------------
// No wait in these libraries is endless. A thread that polls an mbarrier gives up after
// kSpinLimit polls (about a second); it then raises a word, the kernel drains and returns, and
// its outputs are worthless. The word the host reads is one int of device memory per library:
// the caller's (bw_set_failure_word) or, if none was given, one the library allocates at first
// use. bw_device_failure() reads and clears it.
constexpr uint32_t kSpinLimit = 20000000u;

// Polls phase `parity` of the barrier at most `limit` times. False when the limit ran out, or
// when `gave_up` was already raised (by another thread of the block when it points into shared
// memory, by any thread of the launch when it points at the failure word itself); raises
// `gave_up` when it gives up.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t* bar, uint32_t parity, volatile uint32_t* gave_up,
                                                  uint32_t limit = kSpinLimit) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
  for (uint32_t spin = 0; spin < limit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *gave_up) return false;
  }
  *gave_up = 1;
  return false;
}

// The same for a thread with time to spare (a warp that requests copies several stages ahead of
// the warps that use them): between two polls it sleeps, so that its polling takes no issue slots
// and no shared-memory cycles from the warp that shares its scheduler. At most `limit` polls of
// about `nanos` each (about a second with the defaults).
__device__ __forceinline__ bool mbar_wait_bounded_idle(uint64_t* bar, uint32_t parity, volatile uint32_t* gave_up,
                                                       uint32_t nanos = 256u, uint32_t limit = 4000000u) {
  const uint32_t addr = static_cast<uint32_t>(__cvta_generic_to_shared(bar));
  for (uint32_t spin = 0; spin < limit; ++spin) {
    uint32_t done;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    if (done) return true;
    if ((spin & 1023u) == 1023u && *gave_up) return false;
    __nanosleep(nanos);
  }
  *gave_up = 1;
  return false;
}

// The library's failure word (device memory), allocated at first use unless the caller gave
// one; null with the error text set when that allocation failed.
int* failure_word();

// exp(x) written only with IEEE multiply, add and fused multiply-add, each rounded to
// nearest, so that the same sequence on a CPU gives the same bits. The reference calls
// libm's expf (src/kernels.cpp:296,326; src/engine.cpp:56); libm is not reproducible
// across machines, this is. Range reduction x = n*ln2 + r with a two-part ln2, a degree-5
// polynomial for (exp(r) - 1 - r) / r^2 (Cephes expf coefficients), scaling by 2^n through
// the exponent field. Inputs below -87 give 0, above 88 give +inf. Constants are given as
// bit patterns so that no decimal parsing can differ between compilers.
__device__ __forceinline__ float det_expf(float x) {
  if (x < -87.0f) return 0.0f;
  if (x > 88.0f) return __int_as_float(0x7f800000);
  const float t = __fmul_rn(x, __int_as_float(0x3fb8aa3b));           // x * log2(e)
  const float magic = __int_as_float(0x4b400000);                     // 1.5 * 2^23
  const float n = __fsub_rn(__fadd_rn(t, magic), magic);              // round to nearest even
  float r = __fmaf_rn(n, __int_as_float(0xbf318000), x);              // - n * 0.693359375
  r = __fmaf_rn(n, __int_as_float(0x395e8083), r);                    // + n * 2.12194440e-4
  float p = __int_as_float(0x39506967);
  p = __fmaf_rn(p, r, __int_as_float(0x3ab743ce));
  p = __fmaf_rn(p, r, __int_as_float(0x3c088908));
  p = __fmaf_rn(p, r, __int_as_float(0x3d2aa9c1));
  p = __fmaf_rn(p, r, __int_as_float(0x3e2aaaaa));
  p = __fmaf_rn(p, r, __int_as_float(0x3f000000));
  const float z = __fmul_rn(r, r);
  float y = __fmaf_rn(p, z, r);
  y = __fadd_rn(y, 1.0f);
  const int ni = static_cast<int>(n);
  return __fmul_rn(y, __int_as_float((ni + 127) << 23));
}

// The reference's in-vector reduction tree (src/kernels.cpp:57-64): after 16 lane-wise
// chains, s8[i] = l[i] + l[i+8], s4[i] = s8[i] + s8[i+4], then (s4[0]+s4[2]) + (s4[1]+s4[3]).
// Written for one thread that holds all 16 lanes.
__device__ __forceinline__ float tree16(const float* l) {
  float s8[8], s4[4];
#pragma unroll
  for (int i = 0; i < 8; ++i) s8[i] = __fadd_rn(l[i], l[i + 8]);
#pragma unroll
  for (int i = 0; i < 4; ++i) s4[i] = __fadd_rn(s8[i], s8[i + 4]);
  return __fadd_rn(__fadd_rn(s4[0], s4[2]), __fadd_rn(s4[1], s4[3]));
}

// 2^x by the hardware's approximation unit (one instruction; -inf gives 0). The bfloat16
// attention kernels all use this one function for softmax weights and merge factors, so
// they agree bit for bit with each other.
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// SwiGLU of one element for the bfloat16 kernels: (g * sigmoid(g)) * u in float32
// (src/kernels.cpp:291-298) with the hardware's approximate exp2 and reciprocal; the result is
// rounded to bfloat16 by the caller, which hides their last-place error. One definition for
// the stand-alone kernel and the fused epilogues, so all of them give the same bits.
__device__ __forceinline__ float swiglu_one(float g, float u) {
  const float e = __expf(-g);
  const float sig = __fdividef(1.0f, __fadd_rn(1.0f, e));
  return __fmul_rn(__fmul_rn(g, sig), u);
}

// The tail of RMSNorm for one element, and the scale from the sum of squares: one definition
// for the stand-alone kernel and the fused one.
__device__ __forceinline__ float rms_scale(float sumsq, int width, float eps) {
  return __fdiv_rn(1.0f, __fsqrt_rn(__fadd_rn(__fdiv_rn(sumsq, static_cast<float>(width)), eps)));
}
__device__ __forceinline__ float rms_apply(float x, float inv, float w) { return __fmul_rn(__fmul_rn(x, inv), w); }

}  // namespace bw
