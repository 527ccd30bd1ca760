// Argument block shared by the CUDA-core and the tensor-core contraction kernels of the dense layer.
#pragma once
#include "common.cuh"

namespace b200rl {

enum { EPI_FORWARD = 0, EPI_STORE = 1, EPI_ACCUMULATE = 2 };

struct GemmArgs {
    const float* A; long long lda;   // A(m,k)
    const float* B; long long ldb;   // B(n,k)
    int M, N, K;
    int k_per_split;                 // summed-index range handled by one blockIdx.z
    // epilogue
    const float* bias;               // EPI_FORWARD
    float* pre; long long ldpre;     // EPI_FORWARD (nullable)
    float* C; long long ldc;         // output (EPI_FORWARD: y, EPI_STORE: C, EPI_ACCUMULATE with gridDim.z == 1: C += acc)
    float* partial;                  // EPI_ACCUMULATE with gridDim.z > 1: partial[z][M*N] (dense, ld = N)
    int transpose_c;                 // EPI_ACCUMULATE on the tensor-core path only: the result is C^T, i.e. C[n][m] (and partial[z][n][m])
};


// Tensor-core (tcgen05, 3xTF32) version of the same contraction; returns B200RL_ERR_UNSUPPORTED for shapes it does not
// take (the caller then uses the CUDA-core kernel). a_kcontig / b_kcontig: whether the summed index is the contiguous
// one of A(m,k) / B(n,k) in memory. `splits` = number of k ranges (gridDim.z of the CUDA-core kernel).
int launch_gemm_tc(const GemmArgs& a, int epilogue, int activation, bool a_kcontig, bool b_kcontig, int splits, cudaStream_t s, bool b_image = false);

// Operand image of a weight matrix for the tensor-core kernel: B(n, k) = W[n][k] (or W[k][n] when `transposed`) split ONCE into its
// tf32 hi / lo parts and laid out exactly as the kernel's shared-memory B tiles (per 256-row tile and 32-wide k chunk: the swizzled
// hi tile, then the lo tile), so that a CTA brings a chunk's B operand in with one bulk copy instead of loading, splitting and
// storing it again for every row tile. With b_image the kernel takes a.B as such an image (forward and plain-store epilogues,
// k-contiguous A, one k range).
size_t weight_image_bytes(int N, int K);
int launch_weight_image(const float* W, long long ld, int N, int K, bool transposed, float* image, cudaStream_t s);

}  // namespace b200rl
