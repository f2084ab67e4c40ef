// Measurement aid of bench.py, not part of the product library: register-only FP32 FMA loops that
// give the FFMA peak of the device they run on (the roofline denominator of the signature kernels).
// Built by __graft_entry__.build() into libbench_probe.so beside bench.py.
//
//   int64_t psig_probe_fp32_fma(int blocks, int iters, void *scratch, void *stream)
//   int64_t psig_probe_fp32_fma_packed(...)   the same loop as packed two-lane FMAs (fma.rn.f32x2)
//
// Each launches `blocks` x 256 threads that run `iters` x 128 dependent-chain-free FMAs on registers
// only and returns the number of FMAs issued (negative on a bad argument or a failed launch); the
// caller times the launch.  `scratch` must point to at least 4 bytes of device memory.
#include <cuda_runtime.h>
#include <stdint.h>

namespace psig {
namespace {

__global__ void __launch_bounds__(256) ffma_probe(float *out, int iters, float a, float b)
{
    float r[16];
#pragma unroll
    for (int i = 0; i < 16; ++i) r[i] = (float)(threadIdx.x + i) * 1e-3f;
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int rep = 0; rep < 8; ++rep) {
#pragma unroll
            for (int i = 0; i < 16; ++i) r[i] = fmaf(r[i], a, b);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 16; ++i) s += r[i];
    if (s == 12345.678f) out[0] = s;  // keeps the loop alive without a store in practice
}

// Same loop with the packed two-lane FP32 FMA of sm_100 (fma.rn.f32x2): 2 FMAs per instruction.
__global__ void __launch_bounds__(256) ffma2_probe(float *out, int iters, float a, float b)
{
    float2 r[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) r[i] = make_float2((float)(threadIdx.x + i) * 1e-3f, (float)(threadIdx.x - i) * 1e-3f);
    const float2 a2 = make_float2(a, a), b2 = make_float2(b, b);
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int rep = 0; rep < 8; ++rep) {
#pragma unroll
            for (int i = 0; i < 8; ++i) r[i] = __ffma2_rn(r[i], a2, b2);
        }
    }
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) s += r[i].x + r[i].y;
    if (s == 12345.678f) out[0] = s;
}

}  // namespace
}  // namespace psig

extern "C" int64_t psig_probe_fp32_fma(int blocks, int iters, void *scratch, void *stream)
{
    if (blocks <= 0 || iters <= 0 || !scratch) return -4;
    psig::ffma_probe<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float *>(scratch), iters,
                                                                          0.999999f, 1e-7f);
    if (cudaGetLastError() != cudaSuccess) return -7;
    return (int64_t)blocks * 256 * (int64_t)iters * 8 * 16;  // FMAs issued
}

extern "C" int64_t psig_probe_fp32_fma_packed(int blocks, int iters, void *scratch, void *stream)
{
    if (blocks <= 0 || iters <= 0 || !scratch) return -4;
    psig::ffma2_probe<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<float *>(scratch), iters,
                                                                           0.999999f, 1e-7f);
    if (cudaGetLastError() != cudaSuccess) return -7;
    return (int64_t)blocks * 256 * (int64_t)iters * 8 * 16;  // FMAs issued (two per packed instruction)
}
