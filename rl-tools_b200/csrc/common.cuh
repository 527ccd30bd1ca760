// Shared device/host helpers for libb200rl: status handling, activations with the reference's exact definitions,
// launch-geometry constants for B200.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include "../../include/b200rl.h"

namespace b200rl {

constexpr int NUM_SMS = 148;  // B200: 2 dies x 74 SMs; the split heuristics of the planners assume this (they decide scratch sizes, so they must not depend on the device)
constexpr int MAX_DEVICES = 64;

// ordinal of the calling thread's current device, checked against MAX_DEVICES: state that CUDA ties to a device (function attributes,
// events, helper streams, symbol addresses) is kept per ordinal
int current_device(int* device);
// multiprocessor count of the current device (cached per ordinal): the grid of the persistent kernels
int sm_count(int* count);

// records the CUDA error text for b200rl_last_cuda_error() and maps it to a status
int cuda_fail(cudaError_t e, const char* where);
#define B200RL_CUDA_TRY(expr) do { cudaError_t _e = (expr); if(_e != cudaSuccess) return ::b200rl::cuda_fail(_e, #expr); } while(0)
#define B200RL_LAUNCH_CHECK(where) do { cudaError_t _e = cudaPeekAtLastError(); if(_e != cudaSuccess) return ::b200rl::cuda_fail(_e, where); } while(0)

// nn/activation_functions.h:25-55 and math/operations_cuda.h (precise ::tanhf / ::expf, no fast-math intrinsics);
// fast_tanh: math/operations_generic.h:247-251.
__device__ __forceinline__ float fast_tanh_dev(float x){
    x = fminf(fmaxf(x, -3.0f), 3.0f);
    float x2 = x * x;
    return x * (27.0f + x2) / (27.0f + 9.0f * x2);
}
template <int ACT>
__device__ __forceinline__ float activation(float x){
    if constexpr(ACT == B200RL_ACT_IDENTITY) return x;
    else if constexpr(ACT == B200RL_ACT_RELU) return x > 0.0f ? x : 0.0f;
    else if constexpr(ACT == B200RL_ACT_TANH) return tanhf(x);
    else if constexpr(ACT == B200RL_ACT_FAST_TANH) return fast_tanh_dev(x);
    else return 1.0f / (1.0f + expf(-x));
}
// nn/activation_functions.h:57-85
template <int ACT>
__device__ __forceinline__ float d_activation(float x){
    if constexpr(ACT == B200RL_ACT_IDENTITY) return 1.0f;
    else if constexpr(ACT == B200RL_ACT_RELU) return x > 0.0f ? 1.0f : 0.0f;
    else if constexpr(ACT == B200RL_ACT_TANH){ float a = tanhf(x); return 1.0f - a * a; }
    else if constexpr(ACT == B200RL_ACT_FAST_TANH){ float a = fast_tanh_dev(x); return 1.0f - a * a; }
    else { float s = 1.0f / (1.0f + expf(-x)); return s * (1.0f - s); }
}
__device__ __forceinline__ float activation_rt(float x, int act){
    switch(act){
        case B200RL_ACT_IDENTITY: return activation<B200RL_ACT_IDENTITY>(x);
        case B200RL_ACT_RELU: return activation<B200RL_ACT_RELU>(x);
        case B200RL_ACT_TANH: return activation<B200RL_ACT_TANH>(x);
        case B200RL_ACT_FAST_TANH: return activation<B200RL_ACT_FAST_TANH>(x);
        default: return activation<B200RL_ACT_SIGMOID>(x);
    }
}
__device__ __forceinline__ float d_activation_rt(float x, int act){
    switch(act){
        case B200RL_ACT_IDENTITY: return d_activation<B200RL_ACT_IDENTITY>(x);
        case B200RL_ACT_RELU: return d_activation<B200RL_ACT_RELU>(x);
        case B200RL_ACT_TANH: return d_activation<B200RL_ACT_TANH>(x);
        case B200RL_ACT_FAST_TANH: return d_activation<B200RL_ACT_FAST_TANH>(x);
        default: return d_activation<B200RL_ACT_SIGMOID>(x);
    }
}
inline bool valid_activation(int a){ return a >= 0 && a <= B200RL_ACT_SIGMOID; }

// dispatch a runtime activation id to a template argument
#define B200RL_DISPATCH_ACT(act, ...) \
    switch(act){ \
        case B200RL_ACT_IDENTITY: { constexpr int ACT = B200RL_ACT_IDENTITY; __VA_ARGS__; break; } \
        case B200RL_ACT_RELU: { constexpr int ACT = B200RL_ACT_RELU; __VA_ARGS__; break; } \
        case B200RL_ACT_TANH: { constexpr int ACT = B200RL_ACT_TANH; __VA_ARGS__; break; } \
        case B200RL_ACT_FAST_TANH: { constexpr int ACT = B200RL_ACT_FAST_TANH; __VA_ARGS__; break; } \
        default: { constexpr int ACT = B200RL_ACT_SIGMOID; __VA_ARGS__; break; } \
    }

}  // namespace b200rl
