// Measurement aid, built into its own library (libgatzk_b200_tuning.so), not into the
// product: the integer-pipe ceiling of the inner-product arithmetic.  Every lane runs the
// 8x8-limb multiply-accumulate of the packed-evaluation kernel on register operands, with no
// memory traffic; the rate over the whole GPU is the roof the evaluation kernels are
// measured against.
#include <cuda_runtime.h>

#include <cstdint>

#include "../field.cuh"

namespace
{
    constexpr int kThreads = 128;
    constexpr int kAccLimbs = 17;

    template <int CHAINS>
    __global__ void __launch_bounds__(kThreads) mac_peak_kernel(uint32_t iters, uint32_t* sink)
    {
        gzk::WideAcc acc[CHAINS];
        gzk::Fr w, f;
#pragma unroll
        for (int i = 0; i < 8; ++i)
        {
            w.l[i] = threadIdx.x * 2654435761u + i * 40503u + blockIdx.x;
            f.l[i] = threadIdx.x * 2246822519u + i * 3266489917u + 17u;
        }
#pragma unroll
        for (int c = 0; c < CHAINS; ++c) acc[c].clear();
        for (uint32_t it = 0; it < iters; ++it)
        {
#pragma unroll
            for (int c = 0; c < CHAINS; ++c) acc[c].template mac<8>(w.l, f.l);
            w.l[0] += it;  // keep the operands loop-variant
            f.l[7] ^= it;
        }
        uint32_t sum[kAccLimbs];
        uint32_t x = 0;
#pragma unroll
        for (int c = 0; c < CHAINS; ++c)
        {
            acc[c].fold(sum);
#pragma unroll
            for (int i = 0; i < kAccLimbs; ++i) x ^= sum[i];
        }
        if (x == 0x12345678u) sink[0] = x;  // practically never: defeats dead-code elimination
    }
}

// 8x8-limb multiply-accumulates per second over the whole GPU with `chains` (1 or 2)
// independent accumulators per lane.  Returns 0 on success, a cudaError_t value otherwise.
extern "C" int gzk_tuning_mac_peak(int device, int chains, uint32_t iters, double* products_per_second)
{
    if (products_per_second == nullptr) return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t err = cudaSetDevice(device);
    if (err != cudaSuccess) return static_cast<int>(err);
    int sms = 0, nb = 0;
    if ((err = cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, device)) != cudaSuccess) return static_cast<int>(err);
    if (chains == 2)
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, mac_peak_kernel<2>, kThreads, 0);
    else
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, mac_peak_kernel<1>, kThreads, 0);
    if (nb <= 0) nb = 1;
    const unsigned blocks = static_cast<unsigned>(sms * nb);
    uint32_t* sink = nullptr;
    if ((err = cudaMalloc(reinterpret_cast<void**>(&sink), 64)) != cudaSuccess) return static_cast<int>(err);
    cudaEvent_t e0, e1;
    cudaEventCreate(&e0);
    cudaEventCreate(&e1);
    for (int rep = 0; rep < 2; ++rep)
    {
        cudaEventRecord(e0, nullptr);
        if (chains == 2)
            mac_peak_kernel<2><<<blocks, kThreads>>>(iters, sink);
        else
            mac_peak_kernel<1><<<blocks, kThreads>>>(iters, sink);
        cudaEventRecord(e1, nullptr);
        err = cudaDeviceSynchronize();
    }
    float ms = 0.f;
    cudaEventElapsedTime(&ms, e0, e1);
    cudaEventDestroy(e0);
    cudaEventDestroy(e1);
    cudaFree(sink);
    if (err != cudaSuccess) return static_cast<int>(err);
    const double products = static_cast<double>(blocks) * kThreads * static_cast<double>(iters) * (chains == 2 ? 2 : 1);
    *products_per_second = products / (ms * 1e-3);
    return 0;
}
