// Measures rcp.approx.ftz.f32(x) for every x that is exactly a binary16 value and writes the 65536
// results (raw uint32 bit patterns, indexed by the half's bit pattern) to the file named on the
// command line.  CUDA's __half division is built on this instruction (cuda_fp16.hpp, __hdiv), so the
// table lets a CPU restatement of that division reproduce the GPU's bits.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <vector>

__global__ void rcp_kernel(uint32_t *out) {
    const unsigned int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= 65536u) return;
    const float x = __half2float(__ushort_as_half((unsigned short)i));
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    out[i] = __float_as_uint(r);
}

int main(int argc, char **argv) {
    if (argc != 2) {
        std::fprintf(stderr, "usage: %s OUTPUT\n", argv[0]);
        return 2;
    }
    uint32_t *dev = nullptr;
    if (cudaMalloc(&dev, 65536 * sizeof(uint32_t)) != cudaSuccess) return 3;
    rcp_kernel<<<256, 256>>>(dev);
    std::vector<uint32_t> host(65536);
    if (cudaMemcpy(host.data(), dev, 65536 * sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) return 4;
    cudaFree(dev);
    FILE *f = std::fopen(argv[1], "wb");
    if (f == nullptr) return 5;
    std::fwrite(host.data(), sizeof(uint32_t), host.size(), f);
    std::fclose(f);
    return 0;
}
