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
int launch_gemm_tc(const GemmArgs& a, int epilogue, int activation, bool a_kcontig, bool b_kcontig, int splits, cudaStream_t s);

}  // namespace b200rl
