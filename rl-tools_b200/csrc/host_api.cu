// Host-side entry points: status text, the host-buffer rollout pipeline, and reference-compatible random streams
// for the reset table (std::mt19937 + libstdc++'s uniform_real_distribution<float>, as random/operations_cpu.h
// drives them in the reference).
#include "common.cuh"
#include "rollout.cuh"
#include <string.h>
#include <atomic>
#include <mutex>
#include <string>
#include <vector>

namespace b200rl {

static thread_local std::string g_last_cuda_error;
int cuda_fail(cudaError_t e, const char* where){
    g_last_cuda_error = std::string(where) + ": " + cudaGetErrorString(e);
    return B200RL_ERR_CUDA;
}

int current_device(int* device){
    B200RL_CUDA_TRY(cudaGetDevice(device));
    if(*device < 0 || *device >= MAX_DEVICES) return B200RL_ERR_UNSUPPORTED;
    return B200RL_OK;
}
int sm_count(int* count){
    static std::atomic<int> cached[MAX_DEVICES];
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    int n = cached[dev].load(std::memory_order_relaxed);
    if(n == 0){
        B200RL_CUDA_TRY(cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev));
        if(n < 1) return B200RL_ERR_UNSUPPORTED;
        cached[dev].store(n, std::memory_order_relaxed);
    }
    *count = n;
    return B200RL_OK;
}

// ---- MT19937 (Matsumoto & Nishimura), state = 624 words + index ------------------------------------------------
struct Mt { uint32_t* mt; uint32_t& idx; };
static void mt_seed(uint32_t* st, uint32_t seed){
    st[0] = seed;
    for(uint32_t i = 1; i < 624; i++) st[i] = 1812433253u * (st[i - 1] ^ (st[i - 1] >> 30)) + i;
    st[624] = 624;
}
static uint32_t mt_next(uint32_t* st){
    if(st[624] >= 624){
        for(int i = 0; i < 624; i++){
            uint32_t y = (st[i] & 0x80000000u) | (st[(i + 1) % 624] & 0x7fffffffu);
            st[i] = st[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
        }
        st[624] = 0;
    }
    uint32_t y = st[st[624]++];
    y ^= y >> 11; y ^= (y << 7) & 0x9d2c5680u; y ^= (y << 15) & 0xefc60000u; y ^= y >> 18;
    return y;
}
// std::uniform_real_distribution<float>(lo, hi) on mt19937: one draw, float(draw) / 2^32, clamped below 1
static float uniform_real(uint32_t* st, float lo, float hi){
    volatile float u = (float)mt_next(st) / 4294967296.0f;
    if(u >= 1.0f) u = 0.99999994f;
    volatile float scaled = u * (hi - lo);      // volatile: keep multiply and add separately rounded
    return scaled + lo;
}
// A fresh std::normal_distribution<float>(0, 1) per sample (random/operations_cpu.h:40-48): Marsaglia polar method on two
// canonical draws per attempt; the second variate of the pair is discarded.
static float standard_normal(uint32_t* st){
    float x, y, r2;
    do{
        volatile float cx = (float)mt_next(st) / 4294967296.0f; if(cx >= 1.0f) cx = 0.99999994f;
        volatile float cy = (float)mt_next(st) / 4294967296.0f; if(cy >= 1.0f) cy = 0.99999994f;
        volatile float tx = 2.0f * cx, ty = 2.0f * cy;
        x = tx - 1.0f; y = ty - 1.0f;
        volatile float xx = x * x, yy = y * y;
        r2 = xx + yy;
    } while(r2 > 1.0f || r2 == 0.0f);
    volatile float num = -2 * logf(r2);
    const float mult = sqrtf(num / r2);
    return y * mult;
}

// ---- device staging for the host-buffer rollout ---------------------------------------------------------------
struct Staging {
    int device = -1;
    size_t cap_envs = 0, cap_rows = 0, cap_reset = 0;
    float *params = nullptr, *states = nullptr, *episode_return = nullptr, *reset = nullptr, *obs = nullptr, *act = nullptr, *rew = nullptr;
    int32_t* episode_step = nullptr; int32_t* reset_count = nullptr; uint8_t* truncated = nullptr; int* error_flag = nullptr;
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> events;
    void release(){
        float** fp[] = {&params, &states, &episode_return, &reset, &obs, &act, &rew};
        for(auto p : fp){ if(*p) cudaFree(*p); *p = nullptr; }
        if(episode_step) cudaFree(episode_step); episode_step = nullptr;
        if(reset_count) cudaFree(reset_count); reset_count = nullptr;
        if(truncated) cudaFree(truncated); truncated = nullptr;
        if(error_flag) cudaFree(error_flag); error_flag = nullptr;
        if(copy_stream) cudaStreamDestroy(copy_stream); copy_stream = nullptr;
        for(auto e : events) cudaEventDestroy(e);
        events.clear();
        cap_envs = cap_rows = cap_reset = 0; device = -1;
    }
};
// one staging set per device ordinal: a process that drives several GPUs keeps each device's buffers
static Staging g_staging[MAX_DEVICES];
static std::mutex g_staging_mutex;

static int ensure_staging(size_t n_envs, size_t rows, size_t reset_elems, int slabs, Staging** out){
    int dev = 0;
    int rc = current_device(&dev);
    if(rc) return rc;
    Staging& s = g_staging[dev];
    *out = &s;
    s.device = dev;
    if(!s.copy_stream) B200RL_CUDA_TRY(cudaStreamCreateWithFlags(&s.copy_stream, cudaStreamNonBlocking));
    if(!s.params) B200RL_CUDA_TRY(cudaMalloc(&s.params, sizeof(float) * 65536));
    if(!s.error_flag) B200RL_CUDA_TRY(cudaMalloc(&s.error_flag, sizeof(int)));
    if(n_envs > s.cap_envs){
        if(s.states){ cudaFree(s.states); cudaFree(s.episode_return); cudaFree(s.episode_step); cudaFree(s.reset_count); cudaFree(s.truncated); }
        B200RL_CUDA_TRY(cudaMalloc(&s.states, sizeof(float) * 2 * n_envs));
        B200RL_CUDA_TRY(cudaMalloc(&s.episode_return, sizeof(float) * n_envs));
        B200RL_CUDA_TRY(cudaMalloc(&s.episode_step, sizeof(int32_t) * n_envs));
        B200RL_CUDA_TRY(cudaMalloc(&s.reset_count, sizeof(int32_t) * n_envs));
        B200RL_CUDA_TRY(cudaMalloc(&s.truncated, n_envs));
        s.cap_envs = n_envs;
    }
    if(rows > s.cap_rows){
        if(s.obs){ cudaFree(s.obs); cudaFree(s.act); cudaFree(s.rew); }
        B200RL_CUDA_TRY(cudaMalloc(&s.obs, sizeof(float) * 3 * rows));
        B200RL_CUDA_TRY(cudaMalloc(&s.act, sizeof(float) * rows));
        B200RL_CUDA_TRY(cudaMalloc(&s.rew, sizeof(float) * rows));
        s.cap_rows = rows;
    }
    if(reset_elems > s.cap_reset){
        if(s.reset) cudaFree(s.reset);
        B200RL_CUDA_TRY(cudaMalloc(&s.reset, sizeof(float) * reset_elems));
        s.cap_reset = reset_elems;
    }
    while((int)s.events.size() < slabs){
        cudaEvent_t e; B200RL_CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        s.events.push_back(e);
    }
    return B200RL_OK;
}

}  // namespace b200rl
using namespace b200rl;

extern "C" {

int b200rl_version(void){ return 100; }

const char* b200rl_status_string(int status){
    switch(status){
        case B200RL_OK: return "ok";
        case B200RL_ERR_INVALID_ARGUMENT: return "invalid argument";
        case B200RL_ERR_UNSUPPORTED: return "unsupported shape or activation";
        case B200RL_ERR_CUDA: return "CUDA runtime error";
        case B200RL_ERR_DEVICE_FLAG: return "a kernel raised its error flag";
        case B200RL_ERR_SCRATCH_LIMIT: return "problem needs more scratch than the static buffer (B200RL_STATIC_SCRATCH_BYTES) holds";
        default: return "unknown status";
    }
}
const char* b200rl_last_cuda_error(void){ return g_last_cuda_error.c_str(); }

int b200rl_device_malloc(void** ptr, size_t bytes){
    if(!ptr) return B200RL_ERR_INVALID_ARGUMENT;
    B200RL_CUDA_TRY(cudaMalloc(ptr, bytes ? bytes : 1));
    return B200RL_OK;
}
int b200rl_device_free(void* ptr){
    if(ptr) B200RL_CUDA_TRY(cudaFree(ptr));
    return B200RL_OK;
}
static bool memcpy_kind(int kind, cudaMemcpyKind* out){
    if(kind == 0) *out = cudaMemcpyHostToDevice; else if(kind == 1) *out = cudaMemcpyDeviceToHost; else if(kind == 2) *out = cudaMemcpyDeviceToDevice; else return false;
    return true;
}
int b200rl_memcpy(void* dst, const void* src, size_t bytes, int kind, b200rl_stream_t stream){
    cudaMemcpyKind k;
    if(!dst || !src || !memcpy_kind(kind, &k)) return B200RL_ERR_INVALID_ARGUMENT;
    if(bytes == 0) return B200RL_OK;
    B200RL_CUDA_TRY(cudaMemcpyAsync(dst, src, bytes, k, (cudaStream_t)stream));
    if(kind != 2) B200RL_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return B200RL_OK;
}
int b200rl_memcpy_2d(void* dst, size_t dst_pitch_bytes, const void* src, size_t src_pitch_bytes, size_t width_bytes, size_t rows, int kind, b200rl_stream_t stream){
    cudaMemcpyKind k;
    if(!dst || !src || !memcpy_kind(kind, &k) || dst_pitch_bytes < width_bytes || src_pitch_bytes < width_bytes) return B200RL_ERR_INVALID_ARGUMENT;
    if(width_bytes == 0 || rows == 0) return B200RL_OK;
    B200RL_CUDA_TRY(cudaMemcpy2DAsync(dst, dst_pitch_bytes, src, src_pitch_bytes, width_bytes, rows, k, (cudaStream_t)stream));
    if(kind != 2) B200RL_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return B200RL_OK;
}
int b200rl_stream_synchronize(b200rl_stream_t stream){
    B200RL_CUDA_TRY(cudaStreamSynchronize((cudaStream_t)stream));
    return B200RL_OK;
}

int b200rl_rng_init_host(uint32_t* rng_state_host, uint32_t seed){
    if(!rng_state_host) return B200RL_ERR_INVALID_ARGUMENT;
    mt_seed(rng_state_host, seed + 1u);     // random/operations_cpu.h:23
    return B200RL_OK;
}

int b200rl_reset_table_host(uint32_t* rng, int n_envs, int n_steps, const int32_t* episode_step_host, const uint8_t* truncated_host,
                            int step_limit, float* reset_states_host, int n_reset_rounds, int* rounds_used_host){
    if(!rng || !episode_step_host || !truncated_host || !reset_states_host || n_envs < 0 || n_steps < 0 || step_limit < 1 || n_reset_rounds < 0)
        return B200RL_ERR_INVALID_ARGUMENT;
    std::vector<int32_t> es(episode_step_host, episode_step_host + n_envs);
    std::vector<uint8_t> tr(truncated_host, truncated_host + n_envs);
    std::vector<int> cnt(n_envs, 0);
    int used = 0;
    const float PI_F = 3.14159265358979323846f;
    for(int t = 0; t < n_steps; t++){
        for(int e = 0; e < n_envs; e++){
            if(tr[e]){
                if(cnt[e] >= n_reset_rounds) return B200RL_ERR_INVALID_ARGUMENT;
                float* dst = reset_states_host + ((size_t)cnt[e] * n_envs + e) * 2;
                dst[0] = uniform_real(rng, -PI_F, PI_F);      // pendulum/operations_generic.h:57-61: theta first
                dst[1] = uniform_real(rng, -1.0f, 1.0f);
                cnt[e]++; if(cnt[e] > used) used = cnt[e];
                es[e] = 0;
            }
        }
        for(int e = 0; e < n_envs; e++){ es[e] += 1; tr[e] = es[e] == step_limit; }
    }
    if(rounds_used_host) *rounds_used_host = used;
    return B200RL_OK;
}

int b200rl_collect_tables_host(uint32_t* rng, int n_envs, int n_steps, const int32_t* episode_step_host, const uint8_t* truncated_host,
                               int step_limit, float* reset_states_host, int n_reset_rounds, int* rounds_used_host, float* noise_host){
    if(!rng || !episode_step_host || !truncated_host || n_envs < 0 || n_steps < 0 || step_limit < 0 || n_reset_rounds < 0 ||
       (n_reset_rounds > 0 && !reset_states_host) || (!noise_host && n_steps > 0))
        return B200RL_ERR_INVALID_ARGUMENT;
    std::vector<int32_t> es(episode_step_host, episode_step_host + n_envs);
    std::vector<uint8_t> tr(truncated_host, truncated_host + n_envs);
    std::vector<int> cnt(n_envs, 0);
    int used = 0;
    const float PI_F = 3.14159265358979323846f;
    for(int t = 0; t < n_steps; t++){
        for(int e = 0; e < n_envs; e++){              // prologue: on_policy_runner/operations_generic_per_env.h:19-28
            if(tr[e]){
                if(cnt[e] >= n_reset_rounds) return B200RL_ERR_INVALID_ARGUMENT;
                float* dst = reset_states_host + ((size_t)cnt[e] * n_envs + e) * 2;
                dst[0] = uniform_real(rng, -PI_F, PI_F);
                dst[1] = uniform_real(rng, -1.0f, 1.0f);
                cnt[e]++; if(cnt[e] > used) used = cnt[e];
                es[e] = 0;
            }
        }
        for(int e = 0; e < n_envs; e++){              // epilogue: one normal draw per action, :46-60; truncation :72
            noise_host[(size_t)t * n_envs + e] = standard_normal(rng);
            es[e] += 1; tr[e] = step_limit > 0 && es[e] >= step_limit;
        }
    }
    if(rounds_used_host) *rounds_used_host = used;
    return B200RL_OK;
}

// std::uniform_int_distribution on mt19937 for ranges below 2^32 (libstdc++: nearly divisionless bounded draw with a 64-bit product)
static uint32_t uniform_int_below(uint32_t* st, uint32_t range){
    uint64_t product = (uint64_t)mt_next(st) * range;
    uint32_t low = (uint32_t)product;
    if(low < range){
        const uint32_t threshold = (uint32_t)(0u - range) % range;
        while(low < threshold){
            product = (uint64_t)mt_next(st) * range;
            low = (uint32_t)product;
        }
    }
    return (uint32_t)(product >> 32);
}

int b200rl_shuffle_permutation_host(uint32_t* rng, int n_rows, int32_t* perm_host){
    if(!rng || !perm_host || n_rows < 0) return B200RL_ERR_INVALID_ARGUMENT;
    for(int i = 0; i < n_rows; i++) perm_host[i] = i;
    for(int i = 0; i < n_rows; i++){              // rl/algorithms/ppo/operations_generic.h:127-158: swap row i with a row drawn from [i, n-1]
        const int j = i + (int)uniform_int_below(rng, (uint32_t)(n_rows - i));
        const int32_t tmp = perm_host[i]; perm_host[i] = perm_host[j]; perm_host[j] = tmp;
    }
    return B200RL_OK;
}

// gather_batch (rl/components/off_policy_runner/operations_generic.h:413-423, 257-258, 303): per batch element the environment index, then the
// sample offset in [0, eligible - 1] with eligible = full ? capacity : position of that environment's replay buffer
int b200rl_gather_draws_host(uint32_t* rng, int n_envs, int batch, const int32_t* position_host, const uint8_t* full_host, int capacity,
                             int32_t* env_index_host, int32_t* sample_offset_host){
    if(!rng || !position_host || !full_host || !env_index_host || !sample_offset_host || n_envs < 1 || batch < 0 || capacity < 1) return B200RL_ERR_INVALID_ARGUMENT;
    for(int b = 0; b < batch; b++){
        const int e = (int)uniform_int_below(rng, (uint32_t)n_envs);
        const int eligible = full_host[e] ? capacity : position_host[e];
        if(eligible < 1) return B200RL_ERR_INVALID_ARGUMENT;          // the reference requires a non-empty replay buffer (:241)
        env_index_host[b] = e;
        sample_offset_host[b] = (int32_t)uniform_int_below(rng, (uint32_t)eligible);
    }
    return B200RL_OK;
}

// init_weights of a dense layer (nn/layers/dense/operations_generic.h:59-90): per output row the bias draw (when the initialiser
// draws biases) and then the row's input_dim weight draws, all uniform on the host engine; uploaded in two copies.
int b200rl_dense_init_weights(uint32_t* rng, float weight_bound, float bias_bound, int draw_biases, float* W, float* bias,
                              int input_dim, int output_dim, b200rl_stream_t stream){
    if(!rng || !W || !bias || input_dim < 1 || output_dim < 1 || !(weight_bound >= 0.0f) || !(bias_bound >= 0.0f)) return B200RL_ERR_INVALID_ARGUMENT;
    std::vector<float> w((size_t)output_dim * input_dim), b((size_t)output_dim);
    for(int o = 0; o < output_dim; o++){
        b[o] = draw_biases ? uniform_real(rng, -bias_bound, bias_bound) : 0.0f;
        for(int i = 0; i < input_dim; i++) w[(size_t)o * input_dim + i] = uniform_real(rng, -weight_bound, weight_bound);
    }
    cudaStream_t s = (cudaStream_t)stream;
    B200RL_CUDA_TRY(cudaMemcpyAsync(W, w.data(), sizeof(float) * w.size(), cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(bias, b.data(), sizeof(float) * b.size(), cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaStreamSynchronize(s));             // the host vectors go out of scope
    return B200RL_OK;
}

// randn(device, matrix, rng) with the HOST engine (containers/matrix/operations_generic.h:631-639: row-major order, one
// normal_distribution::sample(0, 1) per element), uploaded row by row into a matrix with row pitch ld.
int b200rl_randn_host_rng(uint32_t* rng, float* dst, int ld, int rows, int cols, b200rl_stream_t stream){
    if(!rng || !dst || rows < 0 || cols < 0 || ld < cols) return B200RL_ERR_INVALID_ARGUMENT;
    if(rows == 0 || cols == 0) return B200RL_OK;
    std::vector<float> h((size_t)rows * cols);
    for(size_t i = 0; i < h.size(); i++) h[i] = standard_normal(rng);
    cudaStream_t s = (cudaStream_t)stream;
    B200RL_CUDA_TRY(cudaMemcpy2DAsync(dst, sizeof(float) * (size_t)ld, h.data(), sizeof(float) * (size_t)cols, sizeof(float) * (size_t)cols, (size_t)rows, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaStreamSynchronize(s));
    return B200RL_OK;
}

int b200rl_release_host_staging(void){
    std::lock_guard<std::mutex> lock(g_staging_mutex);
    for(int d = 0; d < MAX_DEVICES; d++) if(g_staging[d].device != -1) g_staging[d].release();
    return B200RL_OK;
}

int b200rl_pendulum_rollout_host(const b200rl_mlp_shape* actor, const float* actor_params_host, float* states_host,
                                 int32_t* episode_step_host, uint8_t* truncated_host, float* episode_return_host,
                                 const float* reset_states_host, int n_reset_rounds, int n_envs, int n_steps, int step_limit,
                                 float* obs_host, float* act_host, float* rew_host, b200rl_stream_t stream){
    int rc = validate_actor(actor);
    if(rc) return rc;
    if(!actor_params_host || !states_host || !episode_step_host || !truncated_host || !episode_return_host || !obs_host || !act_host || !rew_host ||
       n_envs < 0 || n_steps < 0 || n_reset_rounds < 0 || step_limit < 1 || (reset_states_host == nullptr && n_reset_rounds != 0))
        return B200RL_ERR_INVALID_ARGUMENT;
    if(n_envs == 0 || n_steps == 0) return B200RL_OK;
    const size_t N = n_envs, rows = (size_t)n_envs * n_steps, n_params = b200rl_mlp_num_params(actor);
    if(n_params > 65536) return B200RL_ERR_UNSUPPORTED;
    // time slabs: every launch covers all environments (the kernel needs them all in flight to fill the GPU) for a range
    // of steps; the device-to-host copy of slab k (contiguous rows [t0*N, t1*N)) overlaps the kernel of slab k+1
    int slabs = (rows >= (size_t)1 << 20 && n_steps >= 8) ? 8 : 1;
    int slab_steps = (n_steps + slabs - 1) / slabs;
    slabs = (n_steps + slab_steps - 1) / slab_steps;
    std::lock_guard<std::mutex> lock(g_staging_mutex);
    Staging* staging = nullptr;
    rc = ensure_staging(N, rows, (size_t)n_reset_rounds * N * 2, slabs, &staging);
    if(rc) return rc;
    Staging& st = *staging;
    cudaStream_t s = (cudaStream_t)stream;
    B200RL_CUDA_TRY(cudaMemcpyAsync(st.params, actor_params_host, sizeof(float) * n_params, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(st.states, states_host, sizeof(float) * 2 * N, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(st.episode_step, episode_step_host, sizeof(int32_t) * N, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(st.truncated, truncated_host, N, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(st.episode_return, episode_return_host, sizeof(float) * N, cudaMemcpyHostToDevice, s));
    if(n_reset_rounds > 0) B200RL_CUDA_TRY(cudaMemcpyAsync(st.reset, reset_states_host, sizeof(float) * 2 * N * n_reset_rounds, cudaMemcpyHostToDevice, s));
    B200RL_CUDA_TRY(cudaMemsetAsync(st.error_flag, 0, sizeof(int), s));
    B200RL_CUDA_TRY(cudaMemsetAsync(st.reset_count, 0, sizeof(int32_t) * N, s));
    for(int k = 0; k < slabs; k++){
        const int t0 = k * slab_steps, t1 = (t0 + slab_steps < n_steps) ? t0 + slab_steps : n_steps;
        const size_t r0 = (size_t)t0 * N, nr = (size_t)(t1 - t0) * N;
        RolloutArgs a{};
        a.params = st.params; a.states = st.states; a.episode_step = st.episode_step; a.truncated = st.truncated; a.episode_return = st.episode_return;
        a.reset_states = n_reset_rounds > 0 ? st.reset : nullptr; a.n_reset_rounds = n_reset_rounds; a.reset_count = st.reset_count; a.n_envs = n_envs;
        a.env_begin = 0; a.env_count = n_envs;
        a.n_steps = t1 - t0; a.step_limit = step_limit; a.obs = st.obs + r0 * 3; a.act = st.act + r0; a.rew = st.rew + r0; a.error_flag = st.error_flag;
        for(int l = 0; l < 3; l++) a.acts[l] = actor->acts[l];
        rc = rollout_dispatch(actor, a, s);
        if(rc) return rc;
        B200RL_CUDA_TRY(cudaEventRecord(st.events[k], s));
        B200RL_CUDA_TRY(cudaStreamWaitEvent(st.copy_stream, st.events[k], 0));
        B200RL_CUDA_TRY(cudaMemcpyAsync(obs_host + r0 * 3, st.obs + r0 * 3, sizeof(float) * 3 * nr, cudaMemcpyDeviceToHost, st.copy_stream));
        B200RL_CUDA_TRY(cudaMemcpyAsync(act_host + r0, st.act + r0, sizeof(float) * nr, cudaMemcpyDeviceToHost, st.copy_stream));
        B200RL_CUDA_TRY(cudaMemcpyAsync(rew_host + r0, st.rew + r0, sizeof(float) * nr, cudaMemcpyDeviceToHost, st.copy_stream));
    }
    int flag = 0;
    B200RL_CUDA_TRY(cudaMemcpyAsync(states_host, st.states, sizeof(float) * 2 * N, cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(episode_step_host, st.episode_step, sizeof(int32_t) * N, cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(truncated_host, st.truncated, N, cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(episode_return_host, st.episode_return, sizeof(float) * N, cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaMemcpyAsync(&flag, st.error_flag, sizeof(int), cudaMemcpyDeviceToHost, s));
    B200RL_CUDA_TRY(cudaStreamSynchronize(s));
    B200RL_CUDA_TRY(cudaStreamSynchronize(st.copy_stream));
    return flag ? B200RL_ERR_DEVICE_FLAG : B200RL_OK;
}

}
