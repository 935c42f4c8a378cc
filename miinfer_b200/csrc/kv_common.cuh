// Shared device/host helpers of the B200 KV-cache library (CUDA, sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstddef>
#include <cstdint>

#include "b200kv.h"

namespace b200kv {

// ---- status plumbing ---------------------------------------------------------

void set_last_cuda_error(cudaError_t err, const char* where);
int ensure_device();  // B200KV_OK if the current device is sm_100; cached per device

#define B200KV_CUDA_TRY(expr)                                        \
    do {                                                             \
        cudaError_t err__ = (expr);                                  \
        if (err__ != cudaSuccess) {                                  \
            ::b200kv::set_last_cuda_error(err__, #expr);             \
            return B200KV_ERR_CUDA;                                  \
        }                                                            \
    } while (0)

inline bool is_k_q8(uint32_t mode) { return mode == B200KV_Q8_F16 || mode == B200KV_Q8_Q8; }
inline bool is_v_q8(uint32_t mode) { return mode == B200KV_F16_Q8 || mode == B200KV_Q8_Q8; }

// Launch overlap (programmatic dependent launch): 0 = off, n > 0 = on with a guard of n trailing positions.
uint32_t launch_overlap_tail();

// Launches `kernel` on `stream`; with overlap enabled the launch carries the programmatic-stream-serialization
// attribute, so the kernel may become resident before the previous kernel in the stream has finished (it must
// execute griddepcontrol.wait before touching anything that kernel produces).
template <typename... KArgs, typename... Args>
cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, bool allow_overlap,
                          Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    if (allow_overlap && launch_overlap_tail() > 0) {
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = 1;
    }
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// Kernels that need more than 48 KB of dynamic shared memory opt in once PER DEVICE (the attribute belongs to the
// device's context): `done_mask` is the kernel's own bit set of the device ordinals already done.
cudaError_t opt_in_dynamic_smem(const void* kernel, int bytes, std::atomic<uint64_t>& done_mask);

__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Checks the geometry and the pointers a view needs for its mode.
int validate_view(const b200kv_view* view);

// ---- device helpers ------------------------------------------------------------

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Host side: the RoPE constants of a launch -- inv_freq[i] = theta^(-2i/d) for i < d/2 (NeoX) or the step theta^(-2/64)
// of the sectioned form -- kept per thread for the last (theta, d) asked for, so that a decode loop pays the 64-128
// powf calls once and not per launch.
void rope_constants(int rope_mode, float theta, uint32_t head_dim, float* inv_freq, float* sectioned_step);

// sin/cos of an fp32 angle from IEEE double operations only (multiply, fma,
// round-to-integer), so that a host evaluating the same sequence gets the same
// floats: the RoPE trig is part of the bit-exact int8 contract of the append
// kernel, and cosf/sinf differ by ulps between math libraries.  Cody-Waite
// reduction by pi/2 (two-term constant), Taylor series to x^17 / x^16.
__device__ __forceinline__ void sincos_pinned(float angle, float* s_out, float* c_out) {
    const double x = (double)angle;
    const double kd = rint(__dmul_rn(x, 0x1.45f306dc9c883p-1));
    double r = fma(-kd, 0x1.921fb54442d18p+0, x);
    r = fma(-kd, 0x1.1a62633145c07p-54, r);
    const double z = __dmul_rn(r, r);
    double ps = 0x1.952c77030ad4ap-49;
    ps = fma(ps, z, -0x1.ae7f3e733b81fp-41);
    ps = fma(ps, z, 0x1.6124613a86d09p-33);
    ps = fma(ps, z, -0x1.ae64567f544e4p-26);
    ps = fma(ps, z, 0x1.71de3a556c734p-19);
    ps = fma(ps, z, -0x1.a01a01a01a01ap-13);
    ps = fma(ps, z, 0x1.1111111111111p-7);
    ps = fma(ps, z, -0x1.5555555555555p-3);
    const double sr = fma(__dmul_rn(ps, z), r, r);
    double pc = 0x1.ae7f3e733b81fp-45;
    pc = fma(pc, z, -0x1.93974a8c07c9dp-37);
    pc = fma(pc, z, 0x1.1eed8eff8d898p-29);
    pc = fma(pc, z, -0x1.27e4fb7789f5cp-22);
    pc = fma(pc, z, 0x1.a01a01a01a01ap-16);
    pc = fma(pc, z, -0x1.6c16c16c16c17p-10);
    pc = fma(pc, z, 0x1.5555555555555p-5);
    pc = fma(pc, z, -0.5);
    const double cr = fma(pc, z, 1.0);
    const int q = (int)((long long)kd & 3LL);
    double sv = (q & 1) ? cr : sr;
    double cv = (q & 1) ? sr : cr;
    if (q == 2 || q == 3) sv = -sv;
    if (q == 1 || q == 2) cv = -cv;
    *s_out = (float)sv;
    *c_out = (float)cv;
}

}  // namespace b200kv
