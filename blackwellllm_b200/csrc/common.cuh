// Shared helpers for the sm_100a kernels of this engine.
//
// Every launcher is an extern "C" function over raw device pointers and a stream,
// returns 0 on success or a negative BW_ERR_* / positive cudaError_t code, and
// never allocates.  Python binds them with ctypes (kernels/ops.py).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define BW_EXPORT extern "C" __attribute__((visibility("default")))

// error codes returned by launchers (negative: ours; positive: cudaError_t)
#define BW_ERR_BAD_ARG   (-1)
#define BW_ERR_UNSUPPORTED (-2)
#define BW_ERR_DRIVER    (-3)

// element type codes used across the C interface
#define BW_F32  0
#define BW_BF16 1

// activations of feed-forwards (the codes cross the C interface)
//   BW_ACT_SILU           gated:  silu(g) * u
//   BW_ACT_CLAMPED_SWISH  gated:  g' = min(g, limit), u' = clamp(u, -limit, limit):  g' sigmoid(alpha g') (u' + 1)
//   BW_ACT_RELU2          no gate: max(x, 0)^2
//   BW_ACT_GELU_TANH      gated:  0.5 g (1 + tanh(sqrt(2 / pi) (g + 0.044715 g^3))) * u
#define BW_ACT_SILU 0
#define BW_ACT_CLAMPED_SWISH 1
#define BW_ACT_RELU2 2
#define BW_ACT_GELU_TANH 3

// Programmatic dependent launch: a kernel launched through bw::launch may start while the kernel
// before it in the stream is still draining.  Such a kernel calls BW_PDL_TRIGGER() early (the next
// kernel may start launching) and BW_PDL_WAIT() before its first access to memory that an earlier
// kernel may write (everything but weights); the wait returns once all earlier kernels are
// complete and their writes visible.  Both are no-ops for ordinary launches.  BW_PDL=0 in the
// environment turns the early launch off.
#define BW_PDL_TRIGGER() asm volatile("griddepcontrol.launch_dependents;" ::: "memory")
#define BW_PDL_WAIT() asm volatile("griddepcontrol.wait;" ::: "memory")

#define BW_LAUNCH_CHECK() do { cudaError_t e__ = cudaGetLastError(); if (e__ != cudaSuccess) return (int)e__; } while (0)

#include <stdlib.h>
#include <utility>

namespace bw {

inline bool pdl_enabled() {
    static int v = -1;
    if (v < 0) { const char* e = getenv("BW_PDL"); v = (e && e[0] == '0') ? 0 : 1; }
    return v != 0;
}

// overlap == false: an ordinary launch (the kernel starts when everything before it is complete)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_opt(bool overlap, void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                              cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = (overlap && pdl_enabled()) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// the same for a kernel whose CTAs come in clusters of two (grid.x even)
template <typename... KArgs, typename... Args>
inline cudaError_t launch_pairs(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr; cfg.numAttrs = pdl_enabled() ? 2 : 1;
    return cudaLaunchKernelEx(&cfg, kernel, std::forward<Args>(args)...);
}

// The current device's number (0 where none can be asked: host-only use of a planner) and its number of SMs
// (148, the B200's, where none can be asked), looked up once per device.
constexpr int MAX_DEVICES = 64;
inline int current_device() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) { cudaGetLastError(); return 0; }
    return dev;
}
inline int num_sms() {
    static int cached[MAX_DEVICES] = {0};
    const int dev = current_device();
    if (cached[dev] <= 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) { cudaGetLastError(); n = 148; }
        cached[dev] = n;
    }
    return cached[dev];
}
// Raises a kernel's dynamic shared-memory limit once per device (`done`: one flag per device, zero-initialised).
template <typename K>
inline cudaError_t allow_dynamic_smem(K kernel, int bytes, bool (&done)[MAX_DEVICES]) {
    const int dev = current_device();
    if (done[dev]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
    if (e == cudaSuccess) done[dev] = true;
    return e;
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                          Args&&... args) {
    return launch_opt(true, kernel, grid, block, smem, stream, std::forward<Args>(args)...);
}

// The first key position a query at q_pos may see: a sliding window of `window` keys (0: none) and / or
// blocks of `chunk` positions, counted from position 0, that a query does not look out of (0: none).
__host__ __device__ __forceinline__ int first_visible(int q_pos, int window, int chunk) {
    int lo = (window > 0 && q_pos - window + 1 > 0) ? q_pos - window + 1 : 0;
    if (chunk > 0) { const int c0 = q_pos - q_pos % chunk; if (c0 > lo) lo = c0; }
    return lo;
}

// What a query at q_pos sees of the key at k_pos <= q_pos: the keys from first_visible(...) on, and the first
// `keep_first` keys of the sequence whatever the window says (0: none are kept).
__host__ __device__ __forceinline__ bool key_visible(int k_pos, int lo, int keep_first) {
    return k_pos >= lo || k_pos < keep_first;
}

// The distance bias that is taken off a score: r1 ln(1 + r2 (q_pos - k_pos)), r1 and r2 numbers of the query head.
__device__ __forceinline__ float distance_bias(float r1, float r2, int dist) {
    return r1 * log1pf(r2 * (float)dist);
}

// A soft cap on a score: cap * tanh(s / cap).  soft_cap: the library's tanh (the 32-bit path).  soft_cap_fast: tanh as
// 1 - 2 / (2^(2 x log2 e) + 1) with the fast exponential and division; its error is a few ulps of 1, so a few 1e-7 * cap.
__device__ __forceinline__ float soft_cap(float s, float cap) { return cap * tanhf(s / cap); }
__device__ __forceinline__ float soft_cap_fast(float s, float cap, float inv_cap) {
    const float e = exp2f(s * inv_cap * 2.8853900817779268f);
    return cap * (1.f - __fdividef(2.f, e + 1.f));
}

// tanh(x) / x for |x| <= 1 as a polynomial of degree 5 in x^2 (six coefficients fitted over [0, 1]; the error of x * p is
// below 6e-7): five FMAs in place of two special-function instructions.
__device__ __forceinline__ float tanh_over_x_poly(float x2) {
    float p = -0.0030804092530161142f;
    p = fmaf(p, x2, 0.01677677594125271f);
    p = fmaf(p, x2, -0.05163545906543732f);
    p = fmaf(p, x2, 0.13282513618469238f);
    p = fmaf(p, x2, -0.33329179883003235f);
    return fmaf(p, x2, 0.999999463558197f);
}

// A learned bias per (query head, distance): table float32 [heads][len], the last entry standing for every distance
// from len - 1 on.
__device__ __forceinline__ float table_bias(const float* __restrict__ head_row, int len, int dist) {
    return head_row[dist < len ? dist : len - 1];
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);   // lo in the low half
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ float to_f32(float v) { return v; }
__device__ __forceinline__ float to_f32(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float glu(int act, float g, float u, float limit, float alpha) {
    if (act == BW_ACT_CLAMPED_SWISH) {
        g = fminf(g, limit);
        u = fminf(fmaxf(u, -limit), limit);
        return g / (1.f + expf(-alpha * g)) * (u + 1.f);
    }
    if (act == BW_ACT_GELU_TANH) return 0.5f * g * (1.f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g))) * u;
    return g / (1.f + expf(-g)) * u;
}
__device__ __forceinline__ float unary_act(int act, float x) {
    if (act == BW_ACT_RELU2) { const float r = fmaxf(x, 0.f); return r * r; }
    return x;
}

// The output gate of an attention mixer: sigmoid(gate[token, head * dv + c]) for c < dv, 0 for the pad channels beyond
// dv, 1 without a gate.  gate: float32 rows `ld` apart.  dv < 0: the gate has ONE number per head, gate[token, head],
// for the head's first -dv channels.
__device__ __forceinline__ float out_gate(const float* __restrict__ gate, long long ld, int dv, size_t token, int head, int c) {
    if (!gate) return 1.f;
    if (dv < 0) return c < -dv ? 1.f / (1.f + expf(-gate[token * (size_t)ld + (size_t)head])) : 0.f;
    if (c >= dv) return 0.f;
    return 1.f / (1.f + expf(-gate[token * (size_t)ld + (size_t)head * dv + c]));
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

// Block-wide sum in a fixed order (lane tree, then warp 0 over the warp sums), so
// the result for a row never depends on which other rows are in the launch.
// `scratch` holds at least 32 floats.  All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float r = (lane < nwarps) ? scratch[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}

}  // namespace bw
