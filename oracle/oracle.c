/*
 * TEST INFRASTRUCTURE -- CPU oracle for the B200 hot path. NOT part of the shipped library.
 *
 * Plain-C restatement of the reference algorithm (RLtools, header-only C++) for the one path this repository
 * accelerates: dense layer evaluate/forward/backward, MSE gradient, Adam, Pendulum step/reward/observe, the
 * rollout loop that interleaves actor inference with the environment step, and GAE. Every function cites the
 * reference file:line it follows (paths relative to the reference's include/rl_tools/).
 *
 * Only tests/, __graft_entry__.smoke() and bench.py's cpu_baseline / --impl reference legs may load this
 * file's library; the product path never does.
 *
 * Pinning: this restatement is checked bit-for-bit against the real reference compiled from its own headers
 * (oracle/ref_driver.cpp -> oracle/_ref/libref_strict.so, generic CPU device, -O2 -fno-fast-math
 * -ffp-contract=off) by tests/test_oracle_pinning.py (where the reference is present) and against the
 * committed outputs of that same reference build in tests/golden/ (everywhere).
 * Build: gcc -O2 -fno-fast-math -ffp-contract=off -fPIC -shared oracle.c -o _build/liboracle.so -lm
 * The summation order is the reference's generic device order (operations_generic.h), left to right, with
 * separate multiply and add (no fused multiply-add), so results are reproducible across compilers.
 *
 * The reference's random numbers come from libstdc++ (std::mt19937, std::uniform_real_distribution<float>,
 * std::normal_distribution<float>; random/operations_cpu.h:21-48). libstdc++ is not part of the reference
 * tree (GCC 13.3 here); its published algorithms are restated below and pinned against the reference's stream.
 */
#include <stdint.h>
#include <stddef.h>
#include <math.h>
#include <string.h>
#include <stdlib.h>

#define ORC_ACT_IDENTITY 0
#define ORC_ACT_RELU 1
#define ORC_ACT_TANH 2
#define ORC_ACT_FAST_TANH 3
#define ORC_ACT_SIGMOID 4

/* ------------------------------------------------------------------------------------------------------ */
/* RNG: std::mt19937 (MT19937, Matsumoto & Nishimura 1998) seeded as random/operations_cpu.h:21-24 does      */
/* ------------------------------------------------------------------------------------------------------ */
typedef struct { uint32_t mt[624]; int idx; } orc_rng;

/* random/operations_cpu.h:23: engine = mt19937(seed + 1) */
void orc_rng_init(orc_rng* r, uint32_t seed){
    uint32_t s = seed + 1u;
    r->mt[0] = s;
    for(int i = 1; i < 624; i++) r->mt[i] = 1812433253u * (r->mt[i - 1] ^ (r->mt[i - 1] >> 30)) + (uint32_t)i;
    r->idx = 624;
}
uint32_t orc_rng_next(orc_rng* r){
    if(r->idx >= 624){
        for(int i = 0; i < 624; i++){
            uint32_t y = (r->mt[i] & 0x80000000u) | (r->mt[(i + 1) % 624] & 0x7fffffffu);
            r->mt[i] = r->mt[(i + 397) % 624] ^ (y >> 1) ^ ((y & 1u) ? 0x9908b0dfu : 0u);
        }
        r->idx = 0;
    }
    uint32_t y = r->mt[r->idx++];
    y ^= y >> 11; y ^= (y << 7) & 0x9d2c5680u; y ^= (y << 15) & 0xefc60000u; y ^= y >> 18;
    return y;
}
/* std::generate_canonical<float, 24>(mt19937): one 32-bit draw, converted to float (round to nearest),
 * divided by 2^32; a result that rounds up to 1.0f is replaced by the largest float below 1. */
static float orc_canonical(orc_rng* r){
    float sum = (float)orc_rng_next(r);
    float ret = sum / 4294967296.0f;
    if(ret >= 1.0f) ret = nextafterf(1.0f, 0.0f);
    return ret;
}
/* random/operations_cpu.h:32-35 -> std::uniform_real_distribution<float>(lo, hi): u * (hi - lo) + lo */
float orc_uniform_real(orc_rng* r, float lo, float hi){
    return orc_canonical(r) * (hi - lo) + lo;
}
/* The same call with double bounds (the reference writes some bounds as double literals, e.g. rl/environments/acrobot/operations_generic.h:40-43):
 * std::uniform_real_distribution<double> -> std::generate_canonical<double, 53>(mt19937): TWO 32-bit draws, low word first,
 * (g0 + g1 * 2^32) rounded to double, divided by 2^64; then u * (hi - lo) + lo in double. */
double orc_uniform_real_double(orc_rng* r, double lo, double hi){
    double sum = (double)orc_rng_next(r);
    sum += (double)orc_rng_next(r) * 4294967296.0;
    double ret = sum / 18446744073709551616.0;
    if(ret >= 1.0) ret = nextafter(1.0, 0.0);
    return ret * (hi - lo) + lo;
}
/* random/operations_cpu.h:40-48: a FRESH std::normal_distribution<float>(mean, std) per sample, so the second
 * value of the Marsaglia polar pair is always discarded; std == 0 returns mean without consuming the engine. */
float orc_normal(orc_rng* r, float mean, float std){
    if(std == 0) return mean;
    float x, y, r2;
    do{
        x = 2.0f * orc_canonical(r) - 1.0f;
        y = 2.0f * orc_canonical(r) - 1.0f;
        r2 = x * x + y * y;
    } while(r2 > 1.0f || r2 == 0.0f);
    float mult = sqrtf(-2 * logf(r2) / r2);
    float ret = y * mult;
    return ret * std + mean;
}
/* std::uniform_int_distribution<T>(lo, hi) on mt19937 (random/operations_cpu.h:27-29), libstdc++ (GCC >= 11): for a range below
 * 2^32 on a 32-bit generator this is Lemire's nearly divisionless method with a 64-bit product: one draw, redraw while the low half
 * of draw * range falls below (2^32 - range) mod range; the result is the high half. A range of exactly 2^32 values returns the
 * raw draw. Larger ranges (upscaling) do not occur on this path and are not restated. */
uint64_t orc_uniform_int(orc_rng* r, uint64_t lo, uint64_t hi){
    const uint64_t urange = hi - lo;
    if(urange == 0xFFFFFFFFull) return lo + orc_rng_next(r);
    const uint32_t erange = (uint32_t)(urange + 1);
    uint64_t product = (uint64_t)orc_rng_next(r) * erange;
    uint32_t low = (uint32_t)product;
    if(low < erange){
        const uint32_t threshold = (uint32_t)(-erange) % erange;
        while(low < threshold){
            product = (uint64_t)orc_rng_next(r) * erange;
            low = (uint32_t)product;
        }
    }
    return lo + (product >> 32);
}
void orc_rng_uniform_int_stream(uint32_t seed, int n, const uint64_t* lo, const uint64_t* hi, uint64_t* out){
    orc_rng r; orc_rng_init(&r, seed);
    for(int i = 0; i < n; i++) out[i] = orc_uniform_int(&r, lo[i], hi[i]);
}
/* Epoch shuffle of PPO train (rl/algorithms/ppo/operations_generic.h:127-158): for i = 0..n-1 draw j in [i, n-1] and swap rows i
 * and j of the observation, action, advantage, log-prob and target-value columns. perm[i] = the ORIGINAL row that ends up at
 * position i; the engine state advances exactly as in the reference (one draw per row, more on rejection). */
void orc_shuffle_permutation(orc_rng* r, int n, int32_t* perm){
    for(int i = 0; i < n; i++) perm[i] = i;
    for(int i = 0; i < n; i++){
        const int j = (int)orc_uniform_int(r, (uint64_t)i, (uint64_t)(n - 1));
        const int32_t tmp = perm[i]; perm[i] = perm[j]; perm[j] = tmp;
    }
}
void orc_rng_uniform_stream(uint32_t seed, int n, float lo, float hi, float* out){
    orc_rng r; orc_rng_init(&r, seed);
    for(int i = 0; i < n; i++) out[i] = orc_uniform_real(&r, lo, hi);
}
void orc_rng_normal_stream(uint32_t seed, int n, float mean, float std, float* out){
    orc_rng r; orc_rng_init(&r, seed);
    for(int i = 0; i < n; i++) out[i] = orc_normal(&r, mean, std);
}
void orc_rng_mixed_stream(uint32_t seed, int n, const uint8_t* kinds, const float* a, const float* b, float* out){
    orc_rng r; orc_rng_init(&r, seed);
    for(int i = 0; i < n; i++) out[i] = kinds[i] == 0 ? orc_uniform_real(&r, a[i], b[i]) : orc_normal(&r, a[i], b[i]);
}

/* ------------------------------------------------------------------------------------------------------ */
/* activations: nn/activation_functions.h:25-85, math/operations_cpu.h (std:: functions), fast_tanh          */
/* math/operations_generic.h:247-251                                                                        */
/* ------------------------------------------------------------------------------------------------------ */
static float orc_fast_tanh(float x){
    x = x < -3.0f ? -3.0f : (x > 3.0f ? 3.0f : x);
    float x2 = x * x;
    return x * (27 + x2) / (27 + 9 * x2);
}
float orc_activation(float x, int act){
    switch(act){
        case ORC_ACT_IDENTITY: return x;
        case ORC_ACT_RELU: return x > 0.0f ? x : 0.0f;           /* math::max(x, 0) */
        case ORC_ACT_TANH: return tanhf(x);
        case ORC_ACT_FAST_TANH: return orc_fast_tanh(x);
        case ORC_ACT_SIGMOID: return 1.0f / (1.0f + expf(-x));
        default: return 0;
    }
}
float orc_d_activation(float x, int act){
    switch(act){
        case ORC_ACT_IDENTITY: return 1;
        case ORC_ACT_RELU: return x > 0 ? 1 : 0;
        case ORC_ACT_TANH: { float a = tanhf(x); return 1.0f - a * a; }
        case ORC_ACT_FAST_TANH: { float a = orc_fast_tanh(x); return 1.0f - a * a; }
        case ORC_ACT_SIGMOID: { float s = orc_activation(x, ORC_ACT_SIGMOID); return s * (1 - s); }
        default: return 0;
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* dense layer: nn/layers/dense/operations_generic.h                                                         */
/* ------------------------------------------------------------------------------------------------------ */
/* :94-110 evaluate and :112-127 forward: pre = b[o]; pre += W[o][i] * x[b][i] for i ascending; y = act(pre).
 * W is [O,I] row-major, x rows have pitch ldx, pre (optional) pitch ldpre, y pitch ldy. */
void orc_dense_forward(const float* W, const float* bias, const float* x, int ldx, float* pre, int ldpre, float* y, int ldy,
                       int B, int I, int O, int act){
    for(int b = 0; b < B; b++){
        for(int o = 0; o < O; o++){
            float acc = bias[o];
            for(int i = 0; i < I; i++){
                float prod = W[(size_t)o * I + i] * x[(size_t)b * ldx + i];
                acc = acc + prod;
            }
            if(pre) pre[(size_t)b * ldpre + o] = acc;
            y[(size_t)b * ldy + o] = orc_activation(acc, act);
        }
    }
}
/* :167-214 backward / backward_full (and :146-165 backward_input when dW == db == NULL):
 * d_pre = act'(pre) * d_out; db[o] += d_pre; dW[o][i] += d_pre * x[b][i]; d_in[b][i] = sum_o W[o][i] * d_pre,
 * batch outermost, output next, input innermost. Gradients ACCUMULATE. The reference's BLAS/CUDA variants
 * overwrite d_out with d_pre (dense/operations_cpu_blas.h:142-186); store_d_pre reproduces that. */
void orc_dense_backward(const float* W, const float* x, int ldx, const float* pre, int ldpre, float* d_out, int ldd,
                        float* dW, float* db, float* d_in, int ldi, int B, int I, int O, int act, int store_d_pre){
    for(int b = 0; b < B; b++){
        for(int o = 0; o < O; o++){
            float d_pre = orc_d_activation(pre[(size_t)b * ldpre + o], act) * d_out[(size_t)b * ldd + o];
            if(db) db[o] += d_pre;
            for(int i = 0; i < I; i++){
                if(d_in){
                    if(o == 0) d_in[(size_t)b * ldi + i] = 0;
                    float prod = W[(size_t)o * I + i] * d_pre;
                    d_in[(size_t)b * ldi + i] += prod;
                }
                if(dW){
                    float prod = d_pre * x[(size_t)b * ldx + i];
                    dW[(size_t)o * I + i] += prod;
                }
            }
            if(store_d_pre) d_out[(size_t)b * ldd + o] = d_pre;
        }
    }
}

/* nn/loss_functions/mse/operations_generic.h:43-58: d_a = (a - b) * (2 / (rows * cols) * w) */
void orc_mse_gradient(const float* a, int lda, const float* b, int ldb, float* d_a, int ldd, int rows, int cols, float loss_weight){
    float constant = (float)2 / ((float)rows * cols) * loss_weight;
    for(int r = 0; r < rows; r++) for(int c = 0; c < cols; c++){
        float diff = a[(size_t)r * lda + c] - b[(size_t)r * ldb + c];
        d_a[(size_t)r * ldd + c] = diff * constant;
    }
}
/* ------------------------------------------------------------------------------------------------------ */
/* Observation normalisation: rl/components/running_normalizer/operations_generic.h:27-47 (update: per column  */
/* the batch mean and the batch standard deviation about that mean, both by sequential fp32 sums,              */
/* containers/matrix/operations_generic.h:641-650, 674-691: std = 0 if the sum of squares is below 1e-6, else    */
/* sqrt(sum / (rows - 1)); running values move by (batch value - running value) / age),                         */
/* nn/layers/standardize/operations_generic.h:52-66 (set_statistics: precision = std == 0 ? 0 : 1 / std),       */
/* :69-86 (evaluate: (x - mean) * precision, the product skipped where precision is 0). The layer's            */
/* backward_input (:105-124) is not restated: the reference's template does not compile (it names a type its   */
/* specification lacks) and is never reached, the layer being the first of its network.                        */
/* ------------------------------------------------------------------------------------------------------ */
void orc_running_normalizer_update(const float* data, int ld, int rows, int dim, float* mean, float* std, uint64_t* age){
    *age += 1;
    for(int c = 0; c < dim; c++){
        float acc = 0;
        for(int r = 0; r < rows; r++) acc += data[(size_t)r * ld + c];
        const float data_mean = acc / rows;
        float sq = 0;
        for(int r = 0; r < rows; r++){ const float diff = data[(size_t)r * ld + c] - data_mean; sq += diff * diff; }
        const float data_std = sq < 1e-6 ? 0 : sqrtf(sq / (rows - 1));
        mean[c] = mean[c] + (data_mean - mean[c]) / (*age);
        std[c] = std[c] + (data_std - std[c]) / (*age);
    }
}
void orc_standardize_set_statistics(const float* mean, const float* std, int dim, float* layer_mean, float* layer_precision){
    for(int c = 0; c < dim; c++){ layer_mean[c] = mean[c]; layer_precision[c] = std[c] == 0 ? 0 : 1 / std[c]; }
}
void orc_standardize_forward(const float* x, int ldx, const float* mean, const float* precision, float* y, int ldy, int rows, int dim){
    for(int r = 0; r < rows; r++) for(int c = 0; c < dim; c++){
        float v = x[(size_t)r * ldx + c] - mean[c];
        if(precision[c] != 0) v *= precision[c];
        y[(size_t)r * ldy + c] = v;
    }
}
/* Target-network update, utils/polyak/operations_generic.h:10-24 (update) and :26-40 (update_squared):      */
/* target = polyak * target + (1 - polyak) * source [* source], left to right.                                */
void orc_polyak_update(const float* source, int ld_source, float* target, int ld_target, int rows, int cols, float polyak, int square){
    for(int r = 0; r < rows; r++) for(int c = 0; c < cols; c++){
        const float s = source[(size_t)r * ld_source + c];
        float* t = target + (size_t)r * ld_target + c;
        *t = square ? polyak * *t + (1 - polyak) * s * s : polyak * *t + (1 - polyak) * s;
    }
}
/* :9-22 evaluate: sum (a-b)^2 * w / (rows*cols) */
float orc_mse_evaluate(const float* a, int lda, const float* b, int ldb, int rows, int cols, float loss_weight){
    float acc = 0;
    for(int r = 0; r < rows; r++) for(int c = 0; c < cols; c++){
        float diff = a[(size_t)r * lda + c] - b[(size_t)r * ldb + c];
        acc += diff * diff;
    }
    return acc * loss_weight / (rows * cols);
}

/* ------------------------------------------------------------------------------------------------------ */
/* Adam: nn/optimizers/adam/operations_generic.h:49-64, instance/operations_generic.h:25-68,                 */
/* utils/polyak/operations_generic.h:72-88                                                                   */
/* ------------------------------------------------------------------------------------------------------ */
/* _step (:49-59): c1 = 1/(1 - beta1^age), c2 = 1/(1 - beta2^age) via powf, then age++ (age starts at 1). */
void orc_adam_bias_correction(float beta_1, float beta_2, uint32_t* age, float* c1, float* c2){
    uint32_t a = *age;
    *c1 = 1 / (1 - powf(beta_1, (float)a));
    *c2 = 1 / (1 - powf(beta_2, (float)a));
    *age = a + 1;
}
/* update(Adam::Instance) with clipping, weight decay and bias-lr factor off (the defaults):
 *   m = b1*m + (1-b1)*g ; v = b2*v + ((1-b2)*g)*g ; p -= ((alpha*c1)*m) / (sqrt(max(v*c2, eps_sqrt)) + eps) */
void orc_adam_update(float* p, const float* g, float* m, float* v, size_t n,
                     float alpha, float beta_1, float beta_2, float epsilon, float epsilon_sqrt, float c1, float c2){
    for(size_t i = 0; i < n; i++){
        m[i] = beta_1 * m[i] + (1 - beta_1) * g[i];
        v[i] = beta_2 * v[i] + (1 - beta_2) * g[i] * g[i];
        float pre_sqrt = v[i] * c2;
        pre_sqrt = pre_sqrt > epsilon_sqrt ? pre_sqrt : epsilon_sqrt;
        float update = alpha * c1 * m[i] / (sqrtf(pre_sqrt) + epsilon);
        float value = p[i];
        value -= update;
        p[i] = value;
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* MLP on a flat parameter arena. Layout (this repository's, used by oracle and library alike):              */
/* for each layer l: W_l [O_l, I_l] row-major, then b_l [O_l].                                               */
/* nn_models/mlp/operations_generic.h:77-102 (evaluate), :103-120 (forward), :180-204 (backward),            */
/* :152-179 (backward_full), :210-217 (update)                                                               */
/* ------------------------------------------------------------------------------------------------------ */
typedef struct {
    int n_layers;      /* <= 8 */
    int input_dim;
    int dims[8];       /* output dim of each layer */
    int acts[8];
} orc_mlp_shape;

size_t orc_mlp_num_params(const orc_mlp_shape* s){
    size_t n = 0; int in = s->input_dim;
    for(int l = 0; l < s->n_layers; l++){ n += (size_t)s->dims[l] * in + s->dims[l]; in = s->dims[l]; }
    return n;
}
size_t orc_mlp_act_elems(const orc_mlp_shape* s){ size_t n = 0; for(int l = 0; l < s->n_layers; l++) n += s->dims[l]; return n; }

/* evaluate: y [B, O_last] (pitch ldy). scratch-free for the caller: allocates two [B, max_dim] ping-pong buffers. */
void orc_mlp_evaluate(const orc_mlp_shape* s, const float* params, const float* x, int ldx, float* y, int ldy, int B){
    int maxd = 0; for(int l = 0; l < s->n_layers; l++) if(s->dims[l] > maxd) maxd = s->dims[l];
    float* tick = (float*)malloc(sizeof(float) * (size_t)B * maxd);
    float* tock = (float*)malloc(sizeof(float) * (size_t)B * maxd);
    const float* in = x; int ldin = ldx; int I = s->input_dim; const float* p = params;
    for(int l = 0; l < s->n_layers; l++){
        int O = s->dims[l];
        int last = l == s->n_layers - 1;
        float* out = last ? y : ((l % 2 == 0) ? tick : tock);
        int ldo = last ? ldy : O;
        orc_dense_forward(p, p + (size_t)O * I, in, ldin, NULL, 0, out, ldo, B, I, O, s->acts[l]);
        p += (size_t)O * I + O; in = out; ldin = ldo; I = O;
    }
    free(tick); free(tock);
}
/* forward: stores per-layer pre-activations and outputs, concatenated layer after layer, each [B, O_l] dense. */
void orc_mlp_forward(const orc_mlp_shape* s, const float* params, const float* x, int ldx, float* pre, float* out, int B){
    const float* in = x; int ldin = ldx; int I = s->input_dim; const float* p = params;
    for(int l = 0; l < s->n_layers; l++){
        int O = s->dims[l];
        orc_dense_forward(p, p + (size_t)O * I, in, ldin, pre, O, out, O, B, I, O, s->acts[l]);
        p += (size_t)O * I + O; in = out; ldin = O; I = O;
        pre += (size_t)B * O; out += (size_t)B * O;
    }
}
/* backward: d_out [B, O_last] (clobbered), gradients accumulate into grads (same layout as params);
 * d_input optional ([B, input_dim], pitch = input_dim): NULL -> the input layer gets the weights-only backward. */
void orc_mlp_backward(const orc_mlp_shape* s, const float* params, float* grads, const float* x, int ldx,
                      const float* pre, const float* out, float* d_out, float* d_input, int B){
    int L = s->n_layers;
    size_t poff[8], aoff[8]; int Is[8];
    { size_t po = 0, ao = 0; int I = s->input_dim;
      for(int l = 0; l < L; l++){ poff[l] = po; aoff[l] = ao; Is[l] = I; po += (size_t)s->dims[l] * I + s->dims[l]; ao += (size_t)B * s->dims[l]; I = s->dims[l]; } }
    int maxd = s->input_dim; for(int l = 0; l < L; l++) if(s->dims[l] > maxd) maxd = s->dims[l];
    float* tick = (float*)malloc(sizeof(float) * (size_t)B * maxd);
    float* tock = (float*)malloc(sizeof(float) * (size_t)B * maxd);
    float* d_cur = d_out; int ldd = s->dims[L - 1];
    for(int l = L - 1; l >= 0; l--){
        int O = s->dims[l], I = Is[l];
        const float* in = l == 0 ? x : out + aoff[l - 1];
        int ldin = l == 0 ? ldx : I;
        float* d_in = l == 0 ? d_input : ((l % 2 == 0) ? tick : tock);
        const float* W = params + poff[l];
        float* dW = grads + poff[l];
        orc_dense_backward(W, in, ldin, pre + aoff[l], O, d_cur, ldd, dW, dW + (size_t)O * I, d_in, I, B, I, O, s->acts[l], 1);
        d_cur = d_in; ldd = I;
    }
    free(tick); free(tock);
}

/* ------------------------------------------------------------------------------------------------------ */
/* Pendulum: rl/environments/pendulum/pendulum.h:11-25 (parameters), operations_generic.h                    */
/* ------------------------------------------------------------------------------------------------------ */
#define ORC_PI_F 3.141592653589793238462643383279502884f   /* math::PI<float> */
static const float P_G = 10, P_MAX_SPEED = 8, P_MAX_TORQUE = 2, P_DT = 0.05f, P_M = 1, P_L = 1;

static float orc_clip(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }
/* :14-22: f_mod_python(x + pi, 2 pi) - pi with f_mod_python(a, b) = a - b * floor(a / b), all float */
float orc_angle_normalize(float x){
    float a = x + ORC_PI_F, b = 2 * ORC_PI_F;
    return (a - b * floorf(a / b)) - ORC_PI_F;
}
/* :57-61: theta ~ U[-pi, pi] first, then theta_dot ~ U[-1, 1] */
void orc_pendulum_sample_initial_state(orc_rng* r, float* theta, float* theta_dot){
    *theta = orc_uniform_real(r, -ORC_PI_F, ORC_PI_F);
    *theta_dot = orc_uniform_real(r, -1, 1);
}
/* :78-101. The literal 3.0 makes the bracket DOUBLE arithmetic: the float operands are promoted, the sum with
 * theta_dot is formed in double and rounded to float once. */
void orc_pendulum_step(float theta, float theta_dot, float action, float* next_theta, float* next_theta_dot){
    float u_normalised = orc_clip(action, -1, 1);       /* math::clamp */
    float u = P_MAX_TORQUE * u_normalised;
    u = orc_clip(u, -P_MAX_TORQUE, P_MAX_TORQUE);
    float newthdot = theta_dot + (3 * P_G / (2 * P_L) * sinf(theta) + 3.0 / (P_M * P_L * P_L) * u) * P_DT;
    newthdot = orc_clip(newthdot, -P_MAX_SPEED, P_MAX_SPEED);
    float newth = theta + newthdot * P_DT;
    *next_theta = newth; *next_theta_dot = newthdot;
}
/* :130-139: uses the UNCLAMPED action and the PRE-step state; 0.1 and 0.001 are double literals. */
float orc_pendulum_reward(float theta, float theta_dot, float action){
    float angle_norm = orc_angle_normalize(theta);
    float u = P_MAX_TORQUE * action;
    float costs = angle_norm * angle_norm + 0.1 * theta_dot * theta_dot + 0.001 * (u * u);
    return -costs;
}
/* :141-160 ObservationFourier: [cos, sin, theta_dot] */
void orc_pendulum_observe(float theta, float theta_dot, float* obs){
    obs[0] = cosf(theta); obs[1] = sinf(theta); obs[2] = theta_dot;
}
void orc_pendulum_initial_states(uint32_t seed, int n, float* states){
    orc_rng r; orc_rng_init(&r, seed);
    for(int e = 0; e < n; e++) orc_pendulum_sample_initial_state(&r, &states[2 * e], &states[2 * e + 1]);
}
void orc_pendulum_step_batch(int n, const float* states, const float* actions, float* next_states, float* rewards, float* obs, float* next_obs){
    for(int e = 0; e < n; e++){
        orc_pendulum_step(states[2 * e], states[2 * e + 1], actions[e], &next_states[2 * e], &next_states[2 * e + 1]);
        rewards[e] = orc_pendulum_reward(states[2 * e], states[2 * e + 1], actions[e]);
        if(obs) orc_pendulum_observe(states[2 * e], states[2 * e + 1], obs + 3 * e);
        if(next_obs) orc_pendulum_observe(next_states[2 * e], next_states[2 * e + 1], next_obs + 3 * e);
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* AcrobotSwingup: rl/environments/acrobot/acrobot.h:11-27 (parameters: dt 0.2, unit links, torque +-5,        */
/* velocity limits 4 pi / 9 pi), operations_generic.h:46-53 (initial state: theta_1, theta_2 ~ U(-pi, pi),      */
/* velocities 0), :60-99 (dsdt), :101-124 (rk4), :126-151 (step: clamp the action to [-1, 1], scale to the      */
/* torque range, one RK4 step, wrap both angles to [-pi, pi), clamp the velocities), :157-178 (swing-up          */
/* reward on the NEXT state), :180-191 (observation cos / sin of both angles and the two velocities), never     */
/* terminates (:196-199). The float / double mix follows the reference: the unqualified cos / sin calls in      */
/* dsdt take their float argument promoted to double, 2.0 / 6.0 / 1.0 / 0.02 are double literals.               */
/* ------------------------------------------------------------------------------------------------------ */
#define A_DT 0.2f
#define A_MAX_VEL_1 (4 * ORC_PI_F)
#define A_MAX_VEL_2 (9 * ORC_PI_F)
#define A_MIN_TORQUE (-5.0f)
#define A_MAX_TORQUE (5.0f)
#ifndef ORC_ACROBOT_COS
#define ORC_ACROBOT_COS(x) cos(x)
#define ORC_ACROBOT_SIN(x) sin(x)
#endif
static void orc_acrobot_dsdt(const float state[4], float action, float d_state[4]){
    float m1 = 1.0f, m2 = 1.0f, l1 = 1.0f, lc1 = 0.5f, lc2 = 0.5f, I1 = 1.0f, I2 = 1.0f;
    float g = 9.8;
    float theta1 = state[0], theta2 = state[1], dtheta1 = state[2], dtheta2 = state[3];
    float d1 = (m1 * lc1 * lc1 + m2 * (l1 * l1 + lc2 * lc2 + 2 * l1 * lc2 * ORC_ACROBOT_COS(theta2)) + I1 + I2);
    float d2 = m2 * (lc2 * lc2 + l1 * lc2 * ORC_ACROBOT_COS(theta2)) + I2;
    float phi2 = m2 * lc2 * g * cos(theta1 + theta2 - ORC_PI_F / 2.0);
    float phi1 = (-m2 * l1 * lc2 * dtheta2 * dtheta2 * ORC_ACROBOT_SIN(theta2) - 2 * m2 * l1 * lc2 * dtheta2 * dtheta1 * ORC_ACROBOT_SIN(theta2)
                  + (m1 * lc1 + m2 * l1) * g * ORC_ACROBOT_COS(theta1 - ORC_PI_F / 2) + phi2);
    float ddtheta2 = (action + d2 / d1 * phi1 - m2 * l1 * lc2 * dtheta1 * dtheta1 * ORC_ACROBOT_SIN(theta2) - phi2) / (m2 * lc2 * lc2 + I2 - d2 * d2 / d1);
    float ddtheta1 = -(d2 * ddtheta2 + phi1) / d1;
    d_state[0] = dtheta1; d_state[1] = dtheta2; d_state[2] = ddtheta1; d_state[3] = ddtheta2;
}
static void orc_acrobot_rk4(const float state[4], float action, float next_state[4], float dt){
    float k1[4], k2[4], k3[4], k4[4], y1[4], y2[4], y3[4];
    float dt2 = dt / 2.0;
    orc_acrobot_dsdt(state, action, k1);
    for(int i = 0; i < 4; ++i) y1[i] = state[i] + dt2 * k1[i];
    orc_acrobot_dsdt(y1, action, k2);
    for(int i = 0; i < 4; ++i) y2[i] = state[i] + dt2 * k2[i];
    orc_acrobot_dsdt(y2, action, k3);
    for(int i = 0; i < 4; ++i) y3[i] = state[i] + dt * k3[i];
    orc_acrobot_dsdt(y3, action, k4);
    for(int i = 0; i < 4; ++i) next_state[i] = state[i] + dt / 6.0 * (k1[i] + 2 * k2[i] + 2 * k3[i] + k4[i]);
}
static float orc_acrobot_angle_normalize(float x){
    float a = x + ORC_PI_F, b = 2 * ORC_PI_F;
    return (a - b * floorf(a / b)) - ORC_PI_F;
}
void orc_acrobot_step(const float state[4], float action, float next_state[4]){
    float action_clamped = orc_clip(action, -1, 1);
    float action_scaled = (action_clamped + 1.0) / 2.0 * (A_MAX_TORQUE - (A_MIN_TORQUE)) + (A_MIN_TORQUE);
    orc_acrobot_rk4(state, action_scaled, next_state, A_DT);
    next_state[0] = orc_acrobot_angle_normalize(next_state[0]);
    next_state[1] = orc_acrobot_angle_normalize(next_state[1]);
    next_state[2] = orc_clip(next_state[2], -A_MAX_VEL_1, A_MAX_VEL_1);
    next_state[3] = orc_clip(next_state[3], -A_MAX_VEL_2, A_MAX_VEL_2);
}
float orc_acrobot_swingup_reward(const float next_state[4]){
    float a_angle_cost = fabsf(orc_acrobot_angle_normalize(next_state[0] - ORC_PI_F));
    float b_angle_cost = fabsf(orc_acrobot_angle_normalize(next_state[1]));
    return (-a_angle_cost - b_angle_cost) / 100 * A_DT / 0.02;
}
/* the terminating variant (rl::environments::Acrobot): reward -1 per step (:154-156); terminated when the tip is above the bar,
 * (-cos(theta_1) - cos(theta_2 + theta_1)) > 1.0 with the unqualified cos of a float, i.e. in double (:193-195), evaluated on the NEXT
 * state by the runner; initial state: four draws U(-0.1, 0.1) with double bounds, each rounded to float (:38-44) */
int orc_acrobot_terminated(const float state[4]){
    return (-ORC_ACROBOT_COS((double)state[0]) - ORC_ACROBOT_COS((double)(state[1] + state[0]))) > 1.0;
}
void orc_acrobot_terminating_initial_states(uint32_t seed, int n, float* states){
    orc_rng r; orc_rng_init(&r, seed);
    for(int i = 0; i < 4 * n; i++) states[i] = (float)orc_uniform_real_double(&r, -0.1, 0.1);
}
void orc_acrobot_observe(const float state[4], float* obs){
    obs[0] = cosf(state[0]); obs[1] = sinf(state[0]); obs[2] = cosf(state[1]); obs[3] = sinf(state[1]); obs[4] = state[2]; obs[5] = state[3];
}
void orc_acrobot_step_batch(int n, const float* states, const float* actions, float* next_states, float* rewards, float* obs, float* next_obs){
    for(int e = 0; e < n; e++){
        orc_acrobot_step(states + 4 * e, actions[e], next_states + 4 * e);
        rewards[e] = orc_acrobot_swingup_reward(next_states + 4 * e);
        if(obs) orc_acrobot_observe(states + 4 * e, obs + 6 * e);
        if(next_obs) orc_acrobot_observe(next_states + 4 * e, next_obs + 6 * e);
    }
}
/* The rollout of orc_pendulum_rollout for AcrobotSwingup: states [N, 4], observations [T * N, 6], actor 6 -> .. -> 1; a reset takes      */
/* (theta_1, theta_2) from reset_states [R, N, 2] and zeroes the velocities.                                                               */
/* terminating != 0: the terminating variant; a reset then takes all four state components from reset_states [R, N, 4], the reward is -1,  */
/* and `terminated` [T * N] (may be NULL) receives the flag that also ends the episode (per_env.h:93-97).                                 */
int orc_acrobot_rollout_variant(int terminating, const orc_mlp_shape* actor, const float* params, int N, int T, float* states, int32_t* episode_step,
                                uint8_t* truncated, float* episode_return, const float* reset_states, int R, int step_limit,
                                float* obs, float* actions, float* rew, uint8_t* terminated, const float* teacher_states){
    int rc = 0;
    const int D = terminating ? 4 : 2;
    int* reset_count = (int*)calloc((size_t)N, sizeof(int));
    if(actor->input_dim != 6 || actor->dims[actor->n_layers - 1] != 1) { free(reset_count); return -1; }
    for(int t = 0; t < T; t++){
        float* obs_t = obs + (size_t)t * N * 6; float* act_t = actions + (size_t)t * N; float* rew_t = rew + (size_t)t * N;
        if(teacher_states) memcpy(states, teacher_states + (size_t)t * N * 4, sizeof(float) * 4 * (size_t)N);
        for(int e = 0; e < N; e++){
            if(truncated[e]){
                if(reset_count[e] >= R){ rc = -2; continue; }
                for(int k = 0; k < 4; k++) states[4 * e + k] = k < D ? reset_states[((size_t)reset_count[e] * N + e) * D + k] : 0;
                reset_count[e]++; episode_step[e] = 0; episode_return[e] = 0;
            }
            orc_acrobot_observe(states + 4 * e, obs_t + 6 * e);
        }
        orc_mlp_evaluate(actor, params, obs_t, 6, act_t, 1, N);
        for(int e = 0; e < N; e++){
            float ns[4];
            orc_acrobot_step(states + 4 * e, act_t[e], ns);
            float r = terminating ? -1.0f : orc_acrobot_swingup_reward(ns);
            const int term = terminating ? orc_acrobot_terminated(ns) : 0;
            episode_step[e] += 1; episode_return[e] += r;
            truncated[e] = term || (episode_step[e] == step_limit);
            rew_t[e] = r; memcpy(states + 4 * e, ns, sizeof(ns));
            if(terminated) terminated[(size_t)t * N + e] = (uint8_t)term;
        }
    }
    free(reset_count);
    return rc;
}
int orc_acrobot_rollout(const orc_mlp_shape* actor, const float* params, int N, int T, float* states, int32_t* episode_step,
                        uint8_t* truncated, float* episode_return, const float* reset_states, int R, int step_limit,
                        float* obs, float* actions, float* rew, const float* teacher_states){
    return orc_acrobot_rollout_variant(0, actor, params, N, T, states, episode_step, truncated, episode_return, reset_states, R, step_limit, obs, actions, rew, NULL,
                                       teacher_states);
}

/* ------------------------------------------------------------------------------------------------------ */
/* Rollout = off-policy runner step with deterministic actions, repeated T times:                            */
/* rl/components/off_policy_runner/operations_generic_per_env.h:8-66 (prologue: reset-if-truncated, observe), */
/* operations_generic.h:189-205 (interlude: batched policy evaluate), per_env.h:67-108 (epilogue: step,      */
/* reward, counters, truncation). Replay-buffer writes are replaced by flat obs/act/rew outputs, row t*N+e.   */
/* Resets draw from reset_states[k][e] = the k-th reset of env e inside this call (values pre-drawn in the    */
/* reference's draw order by orc_reset_table).                                                               */
/* ------------------------------------------------------------------------------------------------------ */
int orc_pendulum_rollout(const orc_mlp_shape* actor, const float* params, int N, int T, float* states, int32_t* episode_step,
                         uint8_t* truncated, float* episode_return, const float* reset_states, int R, int step_limit,
                         float* obs, float* actions, float* rew, const float* teacher_states){
    int rc = 0;
    int* reset_count = (int*)calloc((size_t)N, sizeof(int));
    if(actor->input_dim != 3 || actor->dims[actor->n_layers - 1] != 1) { free(reset_count); return -1; }
    for(int t = 0; t < T; t++){
        float* obs_t = obs + (size_t)t * N * 3; float* act_t = actions + (size_t)t * N; float* rew_t = rew + (size_t)t * N;
        if(teacher_states) memcpy(states, teacher_states + (size_t)t * N * 2, sizeof(float) * 2 * (size_t)N);
        for(int e = 0; e < N; e++){
            if(truncated[e]){
                if(reset_count[e] >= R){ rc = -2; continue; }
                states[2 * e] = reset_states[((size_t)reset_count[e] * N + e) * 2];
                states[2 * e + 1] = reset_states[((size_t)reset_count[e] * N + e) * 2 + 1];
                reset_count[e]++; episode_step[e] = 0; episode_return[e] = 0;
            }
            orc_pendulum_observe(states[2 * e], states[2 * e + 1], obs_t + 3 * e);
        }
        orc_mlp_evaluate(actor, params, obs_t, 3, act_t, 1, N);
        for(int e = 0; e < N; e++){
            float nt, ntd;
            orc_pendulum_step(states[2 * e], states[2 * e + 1], act_t[e], &nt, &ntd);
            float r = orc_pendulum_reward(states[2 * e], states[2 * e + 1], act_t[e]);
            episode_step[e] += 1; episode_return[e] += r;
            truncated[e] = (episode_step[e] == step_limit);     /* Pendulum never terminates (:243-247) */
            rew_t[e] = r; states[2 * e] = nt; states[2 * e + 1] = ntd;
        }
    }
    free(reset_count);
    return rc;
}
/* Reset table in the reference's draw order: at every step the prologue visits envs 0..N-1 with ONE shared
 * engine (off_policy_runner/operations_cpu.h:46-50) and draws (theta, theta_dot) for each truncated env.
 * Pendulum never terminates, so the truncation schedule depends only on the integer counters. Returns the
 * number of reset rounds written (<= R) or -1 if R is too small. rng state is advanced in place. */
int orc_reset_table(orc_rng* rng, int N, int T, const int32_t* episode_step_in, const uint8_t* truncated_in, int step_limit, float* table, int R){
    int32_t* es = (int32_t*)malloc(sizeof(int32_t) * (size_t)N); uint8_t* tr = (uint8_t*)malloc((size_t)N); int* cnt = (int*)calloc((size_t)N, sizeof(int));
    memcpy(es, episode_step_in, sizeof(int32_t) * (size_t)N); memcpy(tr, truncated_in, (size_t)N);
    int used = 0, rc = 0;
    for(int t = 0; t < T && rc == 0; t++){
        for(int e = 0; e < N; e++){
            if(tr[e]){
                if(cnt[e] >= R){ rc = -1; break; }
                float* dst = table + ((size_t)cnt[e] * N + e) * 2;
                orc_pendulum_sample_initial_state(rng, dst, dst + 1);
                cnt[e]++; if(cnt[e] > used) used = cnt[e];
                es[e] = 0;
            }
        }
        for(int e = 0; e < N; e++){ es[e] += 1; tr[e] = es[e] == step_limit; }
    }
    free(es); free(tr); free(cnt);
    return rc ? rc : used;
}

/* ------------------------------------------------------------------------------------------------------ */
/* GAE: rl/algorithms/ppo/operations_generic.h:59-95. all_values has (steps+1)*N rows, row = step*N + env.    */
/* ------------------------------------------------------------------------------------------------------ */
void orc_gae(const float* rewards, const float* all_values, const uint8_t* terminated, const uint8_t* truncated,
             float* advantages, float* target_values, int N, int steps, float gamma, float lambda, int ignore_termination){
    for(int e = 0; e < N; e++){
        float previous_value = all_values[(size_t)steps * N + e];
        float previous_advantage = 0;
        for(int sf = 0; sf < steps; sf++){
            int sb = steps - 1 - sf;
            size_t pos = (size_t)sb * N + e;
            int term = terminated[pos], trunc = truncated[pos];
            float current = all_values[pos];
            int term_actual = term && !ignore_termination;
            float next = term_actual ? 0 : previous_value;
            float td = rewards[pos] + gamma * next - current;
            if(trunc){ if(!term) td = 0; previous_advantage = 0; }
            float adv = lambda * gamma * previous_advantage + td;
            advantages[pos] = adv;
            target_values[pos] = adv + current;
            previous_advantage = adv; previous_value = current;
        }
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* Diagonal-Gaussian policy head: random/operations_generic.h:87-121 (log_prob and its derivatives).        */
/* neg_log_sqrt_pi is a double expression (-0.5 * log(2 pi)) rounded to float on assignment.                 */
/* ------------------------------------------------------------------------------------------------------ */
float orc_normal_log_prob(float mean, float log_std, float value){
    float neg_log_sqrt_pi = -0.5 * logf(2 * ORC_PI_F);
    float diff = value - mean;
    float std = expf(log_std);
    float pre_square = diff / std;
    return neg_log_sqrt_pi - log_std - 0.5 * pre_square * pre_square;
}
float orc_normal_d_log_prob_d_mean(float mean, float log_std, float value){
    float diff = value - mean; float std = expf(log_std); float pre_square = diff / std;
    return pre_square / std;
}
float orc_normal_d_log_prob_d_log_std(float mean, float log_std, float value){
    float diff = value - mean; float std = expf(log_std); float pre_square = diff / std;
    return -1 + pre_square * pre_square;
}
void orc_normal_functions(int n, const float* mean, const float* log_std, const float* value, float* lp, float* dmean, float* dlogstd){
    for(int i = 0; i < n; i++){
        lp[i] = orc_normal_log_prob(mean[i], log_std[i], value[i]);
        dmean[i] = orc_normal_d_log_prob_d_mean(mean[i], log_std[i], value[i]);
        dlogstd[i] = orc_normal_d_log_prob_d_log_std(mean[i], log_std[i], value[i]);
    }
}

float orc_normal_d_log_prob_d_sample(float mean, float log_std, float value){      /* random/operations_generic.h:114-120 */
    float diff = value - mean; float std = expf(log_std); float pre_square = diff / std;
    return -pre_square / std;
}

/* ------------------------------------------------------------------------------------------------------ */
/* Sample-and-squash layer (the SAC policy head), nn/layers/sample_and_squash/operations_generic.h:            */
/* forward_per_sample :212-260 with external noise: per action dimension log_std clamped to [-20, 2]           */
/* (layer.h:27-36), sample = mean + noise * std, action = tanh(sample),                                         */
/* log_prob += normal log_prob(mean, clamped log_std, sample) - log(1 - action^2 + 1e-6), accumulated in fp32.  */
/* input [B, 2A] = mean | log_std. Outputs: pre_squashing, output [B, A], log_probabilities [B].               */
/* ------------------------------------------------------------------------------------------------------ */
#define ORC_SAS_LOG_STD_LOW (-20.0f)
#define ORC_SAS_LOG_STD_HIGH (2.0f)
#define ORC_SAS_EPS (1e-6f)
static float orc_clampf(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }
void orc_sample_and_squash_forward(const float* input, int ld_in, const float* noise, int B, int A, float* pre_squashing, float* output, float* log_probs){
    for(int b = 0; b < B; b++){
        float log_prob = 0;
        for(int a = 0; a < A; a++){
            const float mean = input[(size_t)b * ld_in + a];
            const float log_std_clipped = orc_clampf(input[(size_t)b * ld_in + A + a], ORC_SAS_LOG_STD_LOW, ORC_SAS_LOG_STD_HIGH);
            const float std = expf(log_std_clipped);
            const float sample = mean + noise[(size_t)b * A + a] * std;
            const float squashed = tanhf(sample);
            pre_squashing[(size_t)b * A + a] = sample;
            output[(size_t)b * A + a] = squashed;
            const float one_minus_square_plus_eps = (1 - squashed * squashed + ORC_SAS_EPS);
            log_prob += orc_normal_log_prob(mean, log_std_clipped, sample) - logf(one_minus_square_plus_eps);
        }
        log_probs[b] = log_prob;
    }
}
/* backward_full_per_sample :290-357 and backward_full :358-398: d_input [B, 2A] from d_output [B, A] (the critic's   */
/* action gradient) plus the entropy term alpha / B * d log_prob; the log_std gradient is zero outside the clamp;        */
/* per-sample d_log_alpha = alpha * (entropy - target_entropy), summed over the batch in order, divided by the number    */
/* of resets (= B for sequence length 1; nn/layers/gru/... num_resets) and ADDED to *log_alpha_gradient.                 */
void orc_sample_and_squash_backward(const float* input, int ld_in, const float* noise, const float* pre_squashing, const float* output, const float* d_output,
                                    float log_alpha, float target_entropy, int B, int A, float* d_input, int ld_din, float* d_log_alpha_per_sample,
                                    float* log_alpha_gradient){
    const float alpha = expf(log_alpha);
    for(int b = 0; b < B; b++){
        float entropy = 0;
        for(int a = 0; a < A; a++){
            const float action = output[(size_t)b * A + a];
            const float d_output_value = d_output[(size_t)b * A + a];
            const float d_tanh_pre_activation = d_output_value * (1 - action * action);
            float d_mu = d_tanh_pre_activation;
            const float nz = noise[(size_t)b * A + a];
            const float d_std = d_tanh_pre_activation * nz;
            const float log_std_pre_clamp = input[(size_t)b * ld_in + A + a];
            const float log_std_clamped = orc_clampf(log_std_pre_clamp, ORC_SAS_LOG_STD_LOW, ORC_SAS_LOG_STD_HIGH);
            const float std = expf(log_std_clamped);
            float d_log_std_clamped = std * d_std;
            const float mu = input[(size_t)b * ld_in + a];
            const float action_sample = pre_squashing[(size_t)b * A + a];
            const float d_log_prob_d_mean = orc_normal_d_log_prob_d_mean(mu, log_std_clamped, action_sample);
            const float d_log_prob_d_sample = orc_normal_d_log_prob_d_sample(mu, log_std_clamped, action_sample);
            d_mu += alpha / B * (d_log_prob_d_mean + d_log_prob_d_sample + 2 * action);
            const float d_log_prob_d_log_std = orc_normal_d_log_prob_d_log_std(mu, log_std_clamped, action_sample);
            d_log_std_clamped += alpha / B * (d_log_prob_d_log_std + d_log_prob_d_sample * nz * std + 2 * action * nz * std);
            const float d_log_std = log_std_pre_clamp < ORC_SAS_LOG_STD_LOW || log_std_pre_clamp > ORC_SAS_LOG_STD_HIGH ? 0 : d_log_std_clamped;
            d_input[(size_t)b * ld_din + a] = d_mu;
            d_input[(size_t)b * ld_din + A + a] = d_log_std;
            const float one_minus_action_square_plus_eps = (1 - action * action + ORC_SAS_EPS);
            const float action_log_prob = orc_normal_log_prob(mu, log_std_clamped, action_sample) - logf(one_minus_action_square_plus_eps);
            entropy += -action_log_prob;
        }
        const float d_alpha = entropy - target_entropy;
        d_log_alpha_per_sample[b] = alpha * d_alpha;
    }
    float d_log_alpha = 0;
    for(int b = 0; b < B; b++) d_log_alpha += d_log_alpha_per_sample[b];
    d_log_alpha /= B;
    *log_alpha_gradient += d_log_alpha;
}

/* ------------------------------------------------------------------------------------------------------ */
/* Off-policy runner step with per-environment replay buffers:                                               */
/* rl/components/off_policy_runner/operations_generic.h:219-238 (step = prologue, interlude, epilogue),       */
/* operations_generic_per_env.h:8-61 (prologue: on truncation draw a new initial state, reset the counters,   */
/* mark the previous transition of a non-empty replay buffer truncated and start a new episode there; then    */
/* observe), :62-108 (epilogue: step, reward, next observation, counters, truncation, replay add),            */
/* rl/components/replay_buffer/operations_generic.h:54-85 (add: row = observation 3, action 1, reward 1, next   */
/* observation 3, terminated, truncated; episode_start[position] = current_episode_start; position wraps;     */
/* a truncated transition starts a new episode at the next position; full once position returns to 0).        */
/* Replay storage: data [N, capacity, 10], episode_start [N, capacity], states / next_states [N, capacity, 2],  */
/* counters [N, 3] = (position, full, current_episode_start). One engine, draws in environment order.          */
/* buf_obs / buf_act / buf_next_obs [N, 3 | 1 | 3]: the runner's step buffers after the last step.             */
/* ------------------------------------------------------------------------------------------------------ */
void orc_offpolicy_steps(const orc_mlp_shape* actor, const float* params, int N, int capacity, int step_limit, int n_steps, orc_rng* rng,
                         float* states, int32_t* episode_step, uint8_t* truncated, float* episode_return,
                         float* replay_data, int64_t* episode_start, float* replay_states, float* replay_next_states, int64_t* counters,
                         float* buf_obs, float* buf_act, float* buf_next_obs){
    for(int s = 0; s < n_steps; s++){
        for(int e = 0; e < N; e++){
            int64_t* cnt = counters + 3 * e;
            if(truncated[e]){
                orc_pendulum_sample_initial_state(rng, &states[2 * e], &states[2 * e + 1]);
                episode_step[e] = 0; episode_return[e] = 0;
                if(cnt[1] || cnt[0] > 0){
                    const int64_t prev = cnt[0] == 0 ? capacity - 1 : cnt[0] - 1;
                    replay_data[((size_t)e * capacity + prev) * 10 + 9] = 1.0f;
                    cnt[2] = cnt[0];
                }
            }
            orc_pendulum_observe(states[2 * e], states[2 * e + 1], buf_obs + 3 * e);
        }
        orc_mlp_evaluate(actor, params, buf_obs, 3, buf_act, 1, N);
        for(int e = 0; e < N; e++){
            int64_t* cnt = counters + 3 * e;
            float nt, ntd;
            orc_pendulum_step(states[2 * e], states[2 * e + 1], buf_act[e], &nt, &ntd);
            const float r = orc_pendulum_reward(states[2 * e], states[2 * e + 1], buf_act[e]);
            orc_pendulum_observe(nt, ntd, buf_next_obs + 3 * e);
            episode_step[e] += 1; episode_return[e] += r;
            const int trunc = episode_step[e] == step_limit;               /* Pendulum never terminates */
            truncated[e] = (uint8_t)trunc;
            const int64_t pos = cnt[0];
            float* row = replay_data + ((size_t)e * capacity + pos) * 10;
            memcpy(row, buf_obs + 3 * e, sizeof(float) * 3); row[3] = buf_act[e]; row[4] = r; memcpy(row + 5, buf_next_obs + 3 * e, sizeof(float) * 3);
            row[8] = 0.0f; row[9] = (float)trunc;
            /* replay_states / replay_next_states stay untouched: in the reference the add() overload for ReplayBufferWithStates names a type
             * (SPEC::T) its specification does not have, so overload resolution silently falls back to the base-class add() (:54-79), which
             * does not store the states. */
            (void)replay_states; (void)replay_next_states;
            episode_start[(size_t)e * capacity + pos] = cnt[2];
            cnt[0] = (pos + 1) % capacity;
            if(trunc) cnt[2] = cnt[0];
            if(cnt[0] == 0 && !cnt[1]) cnt[1] = 1;
            states[2 * e] = nt; states[2 * e + 1] = ntd;
        }
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* Replay-buffer sampling: gather_batch with SEQUENCE_LENGTH 1 (padded length 2),                             */
/* rl/components/off_policy_runner/operations_generic.h:413-423 (per batch element: environment index drawn   */
/* uniformly, then gather_batch_step), :239-411. With the default sampling parameters of sequence length 1    */
/* (off_policy_runner.h:80-87: no random sequence length, no sampling from the initial state) one element is:   */
/* offset ~ U{0 .. eligible - 1} with eligible = full ? capacity : position; index = offset, or                */
/* (position + max_episode_length + offset) mod capacity once the buffer is full (:303-311);                    */
/* sequence step 0 <- observation, action, reward, terminated of that transition; the step is the sequence's   */
/* last (:352), so final_step_mask = 1, sequence step 1 <- its next observation with a zero action (:385-402),  */
/* and next_final_step_mask_base[1] = 1 (:291); reset[0] = next_reset_base[0] = next_reset_base[1] = 1            */
/* (:279-286, 296-302; next_reset views the base from step 1 when the first step is not a target, :85-91).    */
/* Outputs: oa_base [2, batch, 4] (observation 3, action 1), rewards [batch], terminated / reset /             */
/* final_step_mask [batch], next_reset_base / next_final_step_mask_base [2, batch]; env_index / sample_index   */
/* [batch] (optional): which transition was taken. Storage as in orc_offpolicy_steps.                          */
/* ------------------------------------------------------------------------------------------------------ */
void orc_gather_batch(int N, int capacity, int max_episode_length, int batch, orc_rng* rng, const float* replay_data, const int64_t* counters,
                      float* oa_base, float* rewards, uint8_t* terminated, uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask,
                      uint8_t* next_final_step_mask_base, int32_t* env_index, int32_t* sample_index){
    for(int b = 0; b < batch; b++){
        const int e = (int)orc_uniform_int(rng, 0, (uint64_t)(N - 1));
        const int64_t position = counters[3 * e], full = counters[3 * e + 1];
        const int64_t eligible = full ? capacity : position;
        const int64_t offset = (int64_t)orc_uniform_int(rng, 0, (uint64_t)(eligible - 1));
        const int64_t index = full ? (position + max_episode_length + offset) % capacity : offset;
        const float* row = replay_data + ((size_t)e * capacity + index) * 10;
        float* step0 = oa_base + (size_t)b * 4;
        float* step1 = oa_base + ((size_t)batch + b) * 4;
        memcpy(step0, row, sizeof(float) * 4);                 /* observation, action */
        rewards[b] = row[4];
        terminated[b] = row[8] != 0.0f;
        memcpy(step1, row + 5, sizeof(float) * 3);             /* next observation */
        step1[3] = 0.0f;
        reset[b] = 1; final_step_mask[b] = 1;
        next_reset_base[b] = 1; next_reset_base[batch + b] = 1;    /* [1]: through next_reset, the view of steps 1.. (:85-91, :286) */
        next_final_step_mask_base[b] = 0; next_final_step_mask_base[batch + b] = 1;
        if(env_index) env_index[b] = e;
        if(sample_index) sample_index[b] = (int32_t)index;
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* L2F quadrotor, the configuration of the reference's own GPU throughput harness                              */
/* (src/rl/environments/l2f/cuda/benchmark.cu:31-60): state = StateRotors<StateRandomForce<StateBase>>, i.e.   */
/* position 3, orientation quaternion 4 (w first), linear velocity 3, angular velocity 3, a constant            */
/* disturbance force 3 and torque 3, rotor speeds 4 = 23 floats; one step = step()                             */
/* (rl/environments/l2f/operations_generic.h:93-131): the normalised action is clamped to [-1, 1] and mapped to */
/* the rotor-speed range, the state is integrated by one RK4 step (utils/generic/integrators.h:20-49, state    */
/* algebra operations_generic/50_state_algebra.h) of the dynamics (operations_generic/60_dynamics.h:17-110:     */
/* rotor thrust polynomial, thrust and torque sums, quaternion derivative, rotated thrust / mass + gravity,     */
/* Euler's rigid-body equation, disturbance force and torque, first-order rotor response with rising / falling */
/* time constants), then post_integration (operations_generic/70_post_integration.h:17-35, 127-141): quaternion */
/* normalised, position / velocities clamped to the state limits, rotor speeds clamped to the action limits.    */
/* The action noise of the default parameters is 0 (parameters/default.h:64-66), so no draw enters the result.  */
/* dynamics: the 85 floats of parameters.dynamics in declaration order (multirotor.h:22-41). Every expression   */
/* keeps the reference's association (no contraction).                                                          */
/* ------------------------------------------------------------------------------------------------------ */
typedef struct { float position[3], orientation[4], linear_velocity[3], angular_velocity[3], force[3], torque[3], rpm[4]; } orc_l2f_state;
typedef struct { float rotor_positions[4][3], rotor_thrust_directions[4][3], rotor_torque_directions[4][3], rotor_thrust_coefficients[4][3], rotor_torque_constants[4],
                 rotor_time_constants_rising[4], rotor_time_constants_falling[4], mass, gravity[3], J[3][3], J_inv[3][3], hovering_throttle_relative, action_min, action_max; } orc_l2f_dynamics;
static void l2f_cross(const float* a, const float* b, float* out){
    out[0] = a[1] * b[2] - a[2] * b[1]; out[1] = a[2] * b[0] - a[0] * b[2]; out[2] = a[0] * b[1] - a[1] * b[0];
}
static void l2f_matvec(const float A[3][3], const float* v, float* out){
    for(int i = 0; i < 3; i++){ out[i] = 0; for(int j = 0; j < 3; j++) out[i] += A[i][j] * v[j]; }
}
static void l2f_dynamics(const orc_l2f_dynamics* p, const orc_l2f_state* s, const float* setpoint, orc_l2f_state* d){
    float thrust[3] = {0, 0, 0}, torque[3] = {0, 0, 0};
    for(int r = 0; r < 4; r++){                                              /* the rotor speeds in the state drive the body (60_dynamics.h:100) */
        const float rpm = s->rpm[r];
        const float magnitude = p->rotor_thrust_coefficients[r][0] + p->rotor_thrust_coefficients[r][1] * rpm + p->rotor_thrust_coefficients[r][2] * rpm * rpm;
        float rotor_thrust[3];
        for(int i = 0; i < 3; i++){ rotor_thrust[i] = p->rotor_thrust_directions[r][i] * magnitude; thrust[i] += rotor_thrust[i]; }
        const float reaction = magnitude * p->rotor_torque_constants[r];
        for(int i = 0; i < 3; i++) torque[i] += p->rotor_torque_directions[r][i] * reaction;
        const float* a = p->rotor_positions[r];
        torque[0] += a[1] * rotor_thrust[2] - a[2] * rotor_thrust[1];
        torque[1] += a[2] * rotor_thrust[0] - a[0] * rotor_thrust[2];
        torque[2] += a[0] * rotor_thrust[1] - a[1] * rotor_thrust[0];
    }
    for(int i = 0; i < 3; i++) d->position[i] = s->linear_velocity[i];
    const float* q = s->orientation; const float* w = s->angular_velocity;
    d->orientation[0] = -q[1] * w[0] - q[2] * w[1] - q[3] * w[2];
    d->orientation[1] =  q[0] * w[0] + q[2] * w[2] - q[3] * w[1];
    d->orientation[2] =  q[0] * w[1] + q[3] * w[0] - q[1] * w[2];
    d->orientation[3] =  q[0] * w[2] + q[1] * w[1] - q[2] * w[0];
    for(int i = 0; i < 4; i++) d->orientation[i] *= 0.5f;
    float var[3], rotated[3];                                                /* rotate_vector_by_quaternion (quaternion_helper.h:22-36) */
    l2f_cross(q + 1, thrust, var);
    for(int i = 0; i < 3; i++) var[i] *= 2.0f;
    l2f_cross(q + 1, var, rotated);
    for(int i = 0; i < 3; i++) rotated[i] += var[i] * q[0];
    for(int i = 0; i < 3; i++) rotated[i] += thrust[i];
    const float inverse_mass = 1 / p->mass;
    for(int i = 0; i < 3; i++) d->linear_velocity[i] = rotated[i] * inverse_mass;
    for(int i = 0; i < 3; i++) d->linear_velocity[i] += p->gravity[i];
    float v1[3], v2[3];
    l2f_matvec(p->J, w, v1);
    l2f_cross(w, v1, v2);
    for(int i = 0; i < 3; i++) v1[i] = torque[i] - v2[i];
    l2f_matvec(p->J_inv, v1, d->angular_velocity);
    for(int i = 0; i < 3; i++) d->linear_velocity[i] += s->force[i] / p->mass;       /* StateRandomForce, :77-88 */
    float extra[3];
    l2f_matvec(p->J_inv, s->torque, extra);
    for(int i = 0; i < 3; i++) d->angular_velocity[i] += extra[i];
    for(int r = 0; r < 4; r++){                                                      /* StateRotors, :89-101 */
        const float tau = setpoint[r] >= s->rpm[r] ? p->rotor_time_constants_rising[r] : p->rotor_time_constants_falling[r];
        d->rpm[r] = (setpoint[r] - s->rpm[r]) * 1 / tau;
    }
}
static void l2f_axpy(const orc_l2f_state* k, float scalar, orc_l2f_state* out){            /* scalar_multiply_accumulate of the integrated components */
    for(int i = 0; i < 3; i++){
        out->position[i] += scalar * k->position[i]; out->orientation[i] += scalar * k->orientation[i];
        out->linear_velocity[i] += scalar * k->linear_velocity[i]; out->angular_velocity[i] += scalar * k->angular_velocity[i];
    }
    out->orientation[3] += scalar * k->orientation[3];
    for(int i = 0; i < 4; i++) out->rpm[i] += scalar * k->rpm[i];
}
static float l2f_clamp(float x, float lo, float hi){ return x < lo ? lo : (x > hi ? hi : x); }
void orc_l2f_steps(int n, int n_steps, const float* dynamics, float dt, const float* state_limits, const float* states, const float* actions, float* out){
    const orc_l2f_dynamics* p = (const orc_l2f_dynamics*)dynamics;
    for(int e = 0; e < n; e++){
        orc_l2f_state s;
        memcpy(&s, states + (size_t)e * 23, sizeof(s));
        for(int step = 0; step < n_steps; step++){
            float setpoint[4];
            for(int i = 0; i < 4; i++){
                const float half_range = (p->action_max - p->action_min) / 2;
                float a = actions[(size_t)e * 4 + i];
                a += 0.0f;                                                           /* the action noise of the default parameters */
                a = l2f_clamp(a, -1.0f, 1.0f);
                setpoint[i] = a * half_range + p->action_min + half_range;
            }
            orc_l2f_state k1 = s, k2 = s, k3 = s, k4 = s, t;
            l2f_dynamics(p, &s, setpoint, &k1);
            t = s; l2f_axpy(&k1, dt / 2, &t); l2f_dynamics(p, &t, setpoint, &k2);
            t = s; l2f_axpy(&k2, dt / 2, &t); l2f_dynamics(p, &t, setpoint, &k3);
            t = s; l2f_axpy(&k3, dt, &t);     l2f_dynamics(p, &t, setpoint, &k4);
            orc_l2f_state next = s;
            l2f_axpy(&k1, dt / 6, &next); l2f_axpy(&k2, dt / 3, &next); l2f_axpy(&k3, dt / 3, &next); l2f_axpy(&k4, dt / 6, &next);
            float norm = 0;
            for(int i = 0; i < 4; i++) norm += next.orientation[i] * next.orientation[i];
            norm = sqrtf(norm);
            for(int i = 0; i < 4; i++) next.orientation[i] /= norm;
            for(int i = 0; i < 3; i++){
                next.position[i] = l2f_clamp(next.position[i], -state_limits[0], state_limits[0]);
                next.linear_velocity[i] = l2f_clamp(next.linear_velocity[i], -state_limits[1], state_limits[1]);
                next.angular_velocity[i] = l2f_clamp(next.angular_velocity[i], -state_limits[2], state_limits[2]);
            }
            for(int i = 0; i < 4; i++) next.rpm[i] = l2f_clamp(next.rpm[i], p->action_min, p->action_max);
            s = next;                                                               /* force and torque carry over (:142-150) */
        }
        memcpy(out + (size_t)e * 23, &s, sizeof(s));
    }
}

/* L2F as an environment of the runner loop (same configuration): observe (operations_generic/40_observe.h:42-147: position, rotation     */
/* matrix of the quaternion, linear and angular velocity = 18 values; the observation noise of the default parameters is 0), reward          */
/* (parameters/reward_functions/squared/operations_generic.h:12-103 with the desired state at the origin,                                   */
/* operations_generic/35_get_desired_state.h:17-27; the d_action and position-integral components are 0 for this state type), terminated      */
/* (operations_generic.h:143-158, on the NEXT state). mdp = 18 floats: non_negative, scale, constant, termination penalty, the weights         */
/* position, position clip, orientation, linear velocity, angular velocity, linear acceleration, angular acceleration, action, d_action,      */
/* position error integral; termination enabled, position / linear velocity / angular velocity thresholds.                                   */
void orc_l2f_observe(const float* state, float* o){
    const float* q = state + 3;
    for(int i = 0; i < 3; i++) o[i] = state[i] + 0.0f;
    o[3]  = (1 - 2 * q[2] * q[2] - 2 * q[3] * q[3]); o[4]  = (2 * q[1] * q[2] - 2 * q[0] * q[3]); o[5]  = (2 * q[1] * q[3] + 2 * q[0] * q[2]);
    o[6]  = (2 * q[1] * q[2] + 2 * q[0] * q[3]); o[7]  = (1 - 2 * q[1] * q[1] - 2 * q[3] * q[3]); o[8]  = (2 * q[2] * q[3] - 2 * q[0] * q[1]);
    o[9]  = (2 * q[1] * q[3] - 2 * q[0] * q[2]); o[10] = (2 * q[2] * q[3] + 2 * q[0] * q[1]); o[11] = (1 - 2 * q[1] * q[1] - 2 * q[2] * q[2]);
    for(int i = 3; i < 12; i++) o[i] += 0.0f;
    for(int i = 0; i < 3; i++){ o[12 + i] = state[7 + i] + 0.0f; o[15 + i] = state[10 + i] + 0.0f; }
}
int orc_l2f_terminated(const float* mdp, const float* state){
    if(mdp[14] != 0.0f){
        for(int i = 0; i < 3; i++)
            if(fabsf(state[i] - 0) > mdp[15] || fabsf(state[7 + i] - 0) > mdp[16] || fabsf(state[10 + i]) > mdp[17]) return 1;
    }
    return 0;
}
float orc_l2f_reward(const float* dynamics, float dt, const float* mdp, const float* state, const float* action, const float* next){
    const orc_l2f_dynamics* p = (const orc_l2f_dynamics*)dynamics;
    const float orientation_cost = 2 * acosf(1 - fabsf(state[3 + 3]));
    const float x = state[0] - 0, y = state[1] - 0, z = state[2] - 0;
    float position_cost = sqrtf(x * x + y * y + z * z);
    if(mdp[5] > 0) position_cost = position_cost < mdp[5] ? position_cost : mdp[5];
    const float vx = state[7] - 0, vy = state[8] - 0, vz = state[9] - 0;
    const float linear_vel_cost = sqrtf(vx * vx + vy * vy + vz * vz);
    const float angular_vel_cost = sqrtf(state[10] * state[10] + state[11] * state[11] + state[12] * state[12]);
    float la[3], aa[3];
    for(int i = 0; i < 3; i++){ la[i] = next[7 + i] - state[7 + i]; aa[i] = next[10 + i] - state[10 + i]; }
    const float linear_acc_cost = sqrtf(la[0] * la[0] + la[1] * la[1] + la[2] * la[2]) / dt;
    const float angular_acc_cost = sqrtf(aa[0] * aa[0] + aa[1] * aa[1] + aa[2] * aa[2]) / dt;
    float acc = 0;
    for(int i = 0; i < 4; i++){
        const float relative = (action[i] + 1.0f) / 2.0f;
        const float diff = relative - p->hovering_throttle_relative;
        acc += diff * diff;
    }
    float action_cost = sqrtf(acc);
    action_cost *= action_cost;
    float weighted = 0;
    weighted += mdp[4] * position_cost; weighted += mdp[6] * orientation_cost; weighted += mdp[7] * linear_vel_cost; weighted += mdp[8] * angular_vel_cost;
    weighted += mdp[9] * linear_acc_cost; weighted += mdp[10] * angular_acc_cost; weighted += mdp[11] * action_cost; weighted += mdp[12] * 0.0f; weighted += mdp[13] * 0.0f;
    const float scaled = mdp[1] * weighted;
    if(orc_l2f_terminated(mdp, next)) return mdp[3];
    float reward = -scaled + mdp[2];
    return (reward > 0 || mdp[0] == 0.0f) ? reward : 0;
}
void orc_l2f_functions(int n, const float* dynamics, float dt, const float* mdp, const float* states, const float* actions, const float* next_states, float* observations,
                       float* rewards, uint8_t* terminated){
    for(int i = 0; i < n; i++){
        orc_l2f_observe(states + (size_t)i * 23, observations + (size_t)i * 18);
        rewards[i] = orc_l2f_reward(dynamics, dt, mdp, states + (size_t)i * 23, actions + (size_t)i * 4, next_states + (size_t)i * 23);
        terminated[i] = (uint8_t)orc_l2f_terminated(mdp, next_states + (size_t)i * 23);
    }
}
/* The runner loop on the L2F environment (rl/components/off_policy_runner/operations_generic_per_env.h:8-108, as for the other           */
/* environments): per step reset-if-truncated from reset_states [R, N, 23], observe, actor forward (18 -> ... -> 4), step, reward,          */
/* terminated on the next state, counters; an episode ends (truncated) at termination or at step_limit. obs [T * N, 18], act [T * N, 4],     */
/* rew / terminated [T * N], row = step * N + env. Returns 1 if an environment needed more than R resets.                                   */
int orc_l2f_rollout(const orc_mlp_shape* actor, const float* params, const float* dynamics, float dt, const float* state_limits, const float* mdp, int N, int T, float* states,
                    int32_t* episode_step, uint8_t* truncated, float* episode_return, const float* reset_states, int R, int step_limit, float* obs, float* act, float* rew,
                    uint8_t* terminated){
    int rc = 0;
    int* resets = (int*)calloc((size_t)N, sizeof(int));
    for(int t = 0; t < T; t++){
        float* obs_t = obs + (size_t)t * N * 18; float* act_t = act + (size_t)t * N * 4;
        for(int e = 0; e < N; e++){
            if(truncated[e]){
                if(resets[e] < R) memcpy(states + (size_t)e * 23, reset_states + ((size_t)resets[e] * N + e) * 23, sizeof(float) * 23);
                else rc = 1;
                resets[e]++; episode_step[e] = 0; episode_return[e] = 0.0f;
            }
            orc_l2f_observe(states + (size_t)e * 23, obs_t + (size_t)e * 18);
        }
        orc_mlp_evaluate(actor, params, obs_t, 18, act_t, 4, N);
        for(int e = 0; e < N; e++){
            float next[23];
            orc_l2f_steps(1, 1, dynamics, dt, state_limits, states + (size_t)e * 23, act_t + (size_t)e * 4, next);
            const float r = orc_l2f_reward(dynamics, dt, mdp, states + (size_t)e * 23, act_t + (size_t)e * 4, next);
            const int term = orc_l2f_terminated(mdp, next);
            episode_step[e] += 1; episode_return[e] += r;
            truncated[e] = (uint8_t)(term || episode_step[e] == step_limit);
            rew[(size_t)t * N + e] = r; terminated[(size_t)t * N + e] = (uint8_t)term;
            memcpy(states + (size_t)e * 23, next, sizeof(next));
        }
    }
    free(resets);
    return rc;
}

/* ------------------------------------------------------------------------------------------------------ */
/* Replay-buffer sampling for ANY sequence length: gather_batch / gather_batch_step                           */
/* (rl/components/off_policy_runner/operations_generic.h:239-423) with the sampling parameters as flags       */
/* (off_policy_runner.h:80-87; for SEQUENCE_LENGTH > 1 the defaults are all three on):                         */
/*   ORC_GATHER_FROM_INITIAL_STATE  a sequence starts at the first step of the sampled transition's episode   */
/*                                  (episode_start[index], :312-316); the eligible range of a full buffer then */
/*                                  shrinks by max_episode_length (:258)                                        */
/*   ORC_GATHER_RANDOM_LENGTH       sequences are cut to a random length: with probability nominal_probability */
/*                                  (a double draw compared with the float parameter) the nominal length, else  */
/*                                  U{1 .. sequence_length - 1} (:263-272, 361-381)                             */
/*   ORC_GATHER_FIRST_STEP_TARGET   INCLUDE_FIRST_STEP_IN_TARGETS: next_reset views its base from step 0       */
/*                                  instead of step 1 (:85-92), which is where the unconditional write of :286 */
/*                                  lands                                                                       */
/*   ORC_GATHER_DETERMINISTIC       the DETERMINISTIC template flag: environment 0, sample offset = the batch   */
/*                                  element's index instead of draws (:301, :419)                               */
/* Per batch element the padded sequence (sequence_length + 1 steps) is filled by walking the replay buffer:   */
/* after a truncated transition (flag in the buffer, the newest transition, the second to last padded step, or   */
/* a random cut) the next step holds that transition's next observation with a zero action and is marked in     */
/* next_final_step_mask_base, and the step after it starts a new sequence at a new draw. Outputs: oa_base       */
/* [P, batch, 4], rewards / terminated / reset / final_step_mask [L, batch], next_reset_base /                   */
/* next_final_step_mask_base [P, batch] (P = L + 1). Entries the reference leaves unwritten (rewards of padding   */
/* steps, the rows behind a sequence's end) keep what the caller put there.                                      */
/* ------------------------------------------------------------------------------------------------------ */
#define ORC_GATHER_FROM_INITIAL_STATE 1
#define ORC_GATHER_RANDOM_LENGTH 2
#define ORC_GATHER_FIRST_STEP_TARGET 4
#define ORC_GATHER_DETERMINISTIC 8
static int64_t gather_draw_length(orc_rng* rng, int L, float nominal_probability){
    if(orc_uniform_real_double(rng, 0.0, 1.0) < (double)nominal_probability) return L;      /* ENABLE_NOMINAL_SEQUENCE_LENGTH_PROBABILITY (default on) */
    return L > 1 ? (int64_t)orc_uniform_int(rng, 1, (uint64_t)(L - 1)) : L;
}
void orc_gather_batch_sequences(int N, int capacity, int max_episode_length, int batch, int L, int flags, float nominal_probability, orc_rng* rng,
                                const float* replay_data, const int64_t* episode_start, const int64_t* counters, float* oa_base, float* rewards, uint8_t* terminated,
                                uint8_t* reset, uint8_t* next_reset_base, uint8_t* final_step_mask, uint8_t* next_final_step_mask_base){
    const int P = L + 1;
    const int from_initial = flags & ORC_GATHER_FROM_INITIAL_STATE, random_length = flags & ORC_GATHER_RANDOM_LENGTH, deterministic = flags & ORC_GATHER_DETERMINISTIC;
    const int next_offset = (flags & ORC_GATHER_FIRST_STEP_TARGET) ? 0 : 1;
    for(int b = 0; b < batch; b++){
        const int e = deterministic ? 0 : (int)orc_uniform_int(rng, 0, (uint64_t)(N - 1));
        const int64_t position = counters[3 * e], full = counters[3 * e + 1];
        const float* data = replay_data + (size_t)e * capacity * 10;
        const int64_t eligible = full ? (from_initial ? capacity - max_episode_length : capacity) : position;
        int64_t index = 0, length = L, seq_step = 0;
        if(random_length) length = gather_draw_length(rng, L, nominal_probability);
        int previous_truncated = 0, previous_padding = 1;
        for(int q = 0; q < L; q++){ final_step_mask[(size_t)q * batch + b] = 0; reset[(size_t)q * batch + b] = 0; }
        for(int q = 0; q < P; q++){ next_final_step_mask_base[(size_t)q * batch + b] = 0; next_reset_base[(size_t)q * batch + b] = 0; }
        reset[b] = 1; next_reset_base[b] = 1; next_reset_base[(size_t)next_offset * batch + b] = 1;
        for(int q = 0; q < P; q++){
            if(previous_truncated){
                previous_truncated = 0; previous_padding = 1;
                next_final_step_mask_base[(size_t)q * batch + b] = 1;
                if(q < P - 1) reset[(size_t)q * batch + b] = 1;
                continue;
            }
            if(previous_padding){
                if(q < P - 1) reset[(size_t)q * batch + b] = 1;
                next_reset_base[(size_t)q * batch + b] = 1;
                const int64_t offset = deterministic ? b : (int64_t)orc_uniform_int(rng, 0, (uint64_t)(eligible - 1));
                index = full ? (position + max_episode_length + offset) % capacity : offset;
                if(from_initial) index = episode_start[(size_t)e * capacity + index];
            }
            const float* row = data + (size_t)index * 10;
            float* step = oa_base + ((size_t)q * batch + b) * 4;
            memcpy(step, row, sizeof(float) * 4);                                  /* observation, action */
            if(q < P - 1){ rewards[(size_t)q * batch + b] = row[4]; terminated[(size_t)q * batch + b] = row[8] != 0.0f; }
            int truncated = row[9] != 0.0f;
            int64_t next_index = index + 1;
            if(full) next_index %= capacity;
            if(next_index == position) truncated = 1;
            if(q == P - 2) truncated = 1;
            if(random_length){
                if(seq_step == length - 1){
                    truncated = 1;
                    length = L > 1 ? gather_draw_length(rng, L, nominal_probability) : L;      /* :363-377: no draw at sequence length 1 */
                }
                seq_step = truncated ? 0 : seq_step + 1;
            }
            if(truncated && q < P - 1){
                final_step_mask[(size_t)q * batch + b] = 1;
                float* next = oa_base + ((size_t)(q + 1) * batch + b) * 4;
                memcpy(next, row + 5, sizeof(float) * 3);                          /* next observation, zero action */
                next[3] = 0.0f;
            }
            index = next_index;
            previous_padding = 0;
            previous_truncated = truncated;
        }
    }
}

/* ------------------------------------------------------------------------------------------------------ */
/* On-policy collect: rl/components/on_policy_runner/operations_generic.h:105-146 (collect),                  */
/* operations_generic_per_env.h:9-36 (prologue), :37-79 (epilogue), dataset columns on_policy_runner.h:38-72.  */
/* Pendulum: observation 3, action 1 -> row = obs[0:3] action_mean[3] action[4] log_prob[5] reward[6]         */
/* terminated[7] truncated[8] reset[9] value[10] advantage[11] target_value[12]; row index step*N + env;      */
/* reset is truncation delayed by one step: row env of step 0 takes the runner's incoming flag, row pos+N the  */
/* flag after the step at pos. The final observation goes to row T*N + env. params = MLP arena followed by     */
/* log_std[1]. Two sources of randomness: rng != NULL draws inline from ONE engine in the reference's order    */
/* (per step: envs ascending initial states of truncated envs, then envs ascending action noise); rng == NULL  */
/* reads the tables written by orc_collect_tables (reset_states [R,N,2], noise [T,N] standard normal draws).   */
/* step_limit == 0 disables truncation (STEP_LIMIT > 0 && episode_step >= STEP_LIMIT).                        */
/* ------------------------------------------------------------------------------------------------------ */
int orc_pendulum_collect(const orc_mlp_shape* actor, const float* params, int N, int T, float* states, int32_t* episode_step,
                         uint8_t* truncated, float* episode_return, orc_rng* rng, const float* reset_states, int R, const float* noise,
                         int step_limit, float* dataset, int ld){
    if(actor->input_dim != 3 || actor->dims[actor->n_layers - 1] != 1 || ld < 13) return -1;
    const float log_std = params[orc_mlp_num_params(actor)];
    int rc = 0;
    int* reset_count = (int*)calloc((size_t)N, sizeof(int));
    float* obs_t = (float*)malloc(sizeof(float) * 3 * (size_t)N); float* mean_t = (float*)malloc(sizeof(float) * (size_t)N);
    for(int e = 0; e < N; e++) dataset[(size_t)e * ld + 9] = truncated[e] ? 1.0f : 0.0f;
    for(int t = 0; t < T; t++){
        for(int e = 0; e < N; e++){
            if(truncated[e]){
                truncated[e] = 0; episode_step[e] = 0; episode_return[e] = 0;
                if(rng) orc_pendulum_sample_initial_state(rng, &states[2 * e], &states[2 * e + 1]);
                else if(reset_count[e] >= R) rc = -2;
                else{
                    states[2 * e] = reset_states[((size_t)reset_count[e] * N + e) * 2];
                    states[2 * e + 1] = reset_states[((size_t)reset_count[e] * N + e) * 2 + 1];
                    reset_count[e]++;
                }
            }
            orc_pendulum_observe(states[2 * e], states[2 * e + 1], obs_t + 3 * e);
            memcpy(dataset + ((size_t)t * N + e) * ld, obs_t + 3 * e, sizeof(float) * 3);
        }
        orc_mlp_evaluate(actor, params, obs_t, 3, mean_t, 1, N);
        for(int e = 0; e < N; e++){
            float* row = dataset + ((size_t)t * N + e) * ld;
            const float mean = mean_t[e];
            const float std = expf(log_std);
            const float action = rng ? orc_normal(rng, mean, std) : noise[(size_t)t * N + e] * std + mean;
            row[3] = mean; row[4] = action; row[5] = 0 + orc_normal_log_prob(mean, log_std, action);
            float nt, ntd;
            orc_pendulum_step(states[2 * e], states[2 * e + 1], action, &nt, &ntd);
            const float r = orc_pendulum_reward(states[2 * e], states[2 * e + 1], action);
            row[7] = 0;                                        /* Pendulum never terminates */
            episode_return[e] += r; row[6] = r;
            episode_step[e] += 1;
            const int trunc = step_limit > 0 && episode_step[e] >= step_limit;
            row[8] = (float)trunc;
            row[(size_t)N * ld + 9] = (float)trunc;
            truncated[e] = (uint8_t)trunc;
            states[2 * e] = nt; states[2 * e + 1] = ntd;
        }
    }
    for(int e = 0; e < N; e++) orc_pendulum_observe(states[2 * e], states[2 * e + 1], dataset + ((size_t)T * N + e) * ld);
    free(reset_count); free(obs_t); free(mean_t);
    return rc;
}
/* The draws of one collect call as tables, in the engine order described above. The truncation schedule depends only on
 * the integer counters (Pendulum never terminates). noise holds the standard-normal variate of each fresh
 * std::normal_distribution (action = noise * std + mean). Returns the number of reset rounds used or -1 if R is too small. */
int orc_collect_tables(orc_rng* rng, int N, int T, const int32_t* episode_step_in, const uint8_t* truncated_in, int step_limit,
                       float* reset_states, int R, float* noise){
    int32_t* es = (int32_t*)malloc(sizeof(int32_t) * (size_t)N); uint8_t* tr = (uint8_t*)malloc((size_t)N); int* cnt = (int*)calloc((size_t)N, sizeof(int));
    memcpy(es, episode_step_in, sizeof(int32_t) * (size_t)N); memcpy(tr, truncated_in, (size_t)N);
    int used = 0, rc = 0;
    for(int t = 0; t < T && rc == 0; t++){
        for(int e = 0; e < N; e++){
            if(tr[e]){
                if(cnt[e] >= R){ rc = -1; break; }
                float* dst = reset_states + ((size_t)cnt[e] * N + e) * 2;
                orc_pendulum_sample_initial_state(rng, dst, dst + 1);
                cnt[e]++; if(cnt[e] > used) used = cnt[e];
                es[e] = 0;
            }
        }
        if(rc) break;
        for(int e = 0; e < N; e++){
            noise[(size_t)t * N + e] = orc_normal(rng, 0.0f, 1.0f);
            es[e] += 1; tr[e] = step_limit > 0 && es[e] >= step_limit;
        }
    }
    free(es); free(tr); free(cnt);
    return rc ? rc : used;
}

/* ------------------------------------------------------------------------------------------------------ */
/* PPO minibatch loss gradient w.r.t. the actor output and log_std: rl/algorithms/ppo/operations_generic.h   */
/* :173-184 (advantage mean / std over the minibatch), :214-296 (per-sample clipped surrogate gradient,      */
/* entropy bonus, log_std gradient accumulation). Default parameters (rl/algorithms/ppo/ppo.h:13-38).        */
/* current_actions [B,A] = actor(obs) with the current parameters; rollout_actions [B,A], rollout_log_probs  */
/* [B], advantages [B] from the dataset; d_actions [B,A] receives d loss / d actor output; d_log_std [A]      */
/* ACCUMULATES (the reference increments log_std.gradient, zeroed by zero_gradient before).                  */
/* ------------------------------------------------------------------------------------------------------ */
void orc_ppo_policy_gradient(const float* current_actions, const float* rollout_actions, const float* log_std, const float* rollout_log_probs,
                             const float* advantages, float* d_actions, float* d_log_std, int B, int A,
                             float epsilon_clip, float entropy_coefficient, float advantage_epsilon, int normalize_advantage, int learn_action_std){
    float advantage_mean = 0, advantage_std = 0;
    if(normalize_advantage){
        for(int b = 0; b < B; b++){ float a = advantages[b]; advantage_mean += a; advantage_std += a * a; }
        advantage_mean /= B; advantage_std /= B;
        float var = advantage_std - advantage_mean * advantage_mean;
        advantage_std = sqrtf(var > 0 ? var : 0);
    }
    float* d_lp_d_logstd = (float*)malloc(sizeof(float) * (size_t)A);
    for(int b = 0; b < B; b++){
        float action_log_prob = 0;
        for(int i = 0; i < A; i++){
            float cur = current_actions[(size_t)b * A + i], roll = rollout_actions[(size_t)b * A + i], ls = log_std[i];
            action_log_prob += orc_normal_log_prob(cur, ls, roll);
            d_actions[(size_t)b * A + i] = orc_normal_d_log_prob_d_mean(cur, ls, roll);
            if(learn_action_std){
                float d_entropy = -(float)1 / B * entropy_coefficient;
                d_log_std[i] += d_entropy;
                d_lp_d_logstd[i] = orc_normal_d_log_prob_d_log_std(cur, ls, roll);
            }
        }
        float advantage = advantages[b];
        if(normalize_advantage) advantage = (advantage - advantage_mean) / (advantage_std + advantage_epsilon);
        float log_ratio = action_log_prob - rollout_log_probs[b];
        float ratio = expf(log_ratio);
        float lo = 1 - epsilon_clip, hi = 1 + epsilon_clip;
        float clipped_ratio = ratio < lo ? lo : (ratio > hi ? hi : ratio);
        int clipped = ratio != clipped_ratio;
        float normal_advantage = ratio * advantage, clipped_advantage = clipped_ratio * advantage;
        int ratio_min_switch = normal_advantage - clipped_advantage <= 0.0f;
        float d_loss_d_surrogate = -(float)1 / B;
        float d_surrogate_d_ratio = (ratio_min_switch ? 1.0f : 0.0f) * advantage + (ratio_min_switch ? 0.0f : 1.0f) * advantage * (clipped ? 0.0f : 1.0f);
        float d_loss_d_ratio = d_loss_d_surrogate * d_surrogate_d_ratio;
        float d_loss_d_lp = d_loss_d_ratio * ratio;
        for(int i = 0; i < A; i++){
            d_actions[(size_t)b * A + i] *= d_loss_d_lp;
            if(learn_action_std) d_log_std[i] += d_loss_d_lp * d_lp_d_logstd[i];
        }
    }
    free(d_lp_d_logstd);
}

/* ---- L2F initial state (rl/environments/l2f/operations_generic/30_sample_initial_state.h:19-207, the harness' state StateRotors<StateRandomForce<StateBase>>) ---- */
/* init: guidance, max_position, max_angle, max_linear_velocity, max_angular_velocity, relative_rpm, min_rpm, max_rpm, force mean / std, torque mean / std.        */
/* The state as a function of its draws: u[17] canonical uniforms in [0, 1) (guidance; position 3; orientation u, v, angle; linear velocity 3; angular velocity 3;  */
/* rotor speeds 4) and nrm[6] standard normals (force 3, torque 3; the third torque component has std / 100). uniform(lo, hi) = u * (hi - lo) + lo, normal =       */
/* n * std + mean (std == 0: the mean); the reference writes 2.0 / 1.0 / 0.5 as double literals in sample_orientation, so those products are taken in double.      */
void orc_l2f_initial_state_from_draws(const float* init, float action_min, float action_max, const float* u, const float* nrm, float* state){
    const int guidance = u[0] < init[0];
    float* position = state; float* q = state + 3; float* lin = state + 7; float* ang = state + 10; float* force = state + 13; float* torque = state + 16; float* rpm = state + 19;
    for(int i = 0; i < 3; i++) position[i] = guidance ? 0.0f : u[1 + i] * (init[1] - (-init[1])) + (-init[1]);
    if(init[2] > 0 && !guidance){
        const float uu = u[4], v = u[5], angle = u[6];
        const float phi = (float)(2.0 * (double)3.14159265358979323846f * (double)uu);
        const float cos_theta = (float)(1.0 - 2.0 * (double)v);
        const float sin_theta = (float)sqrt(1.0 - (double)(cos_theta * cos_theta));
        const float x = sin_theta * cosf(phi), y = sin_theta * sinf(phi), z = cos_theta;
        const float half = (float)(0.5 * (double)angle);
        const float sn = sinf(half);
        q[0] = cosf(half); q[1] = x * sn; q[2] = y * sn; q[3] = z * sn;
    }
    else { q[0] = 1; q[1] = 0; q[2] = 0; q[3] = 0; }
    for(int i = 0; i < 3; i++){
        lin[i] = guidance ? 0.0f : u[7 + i] * (init[3] - (-init[3])) + (-init[3]);
        ang[i] = guidance ? 0.0f : u[10 + i] * (init[4] - (-init[4])) + (-init[4]);
    }
    for(int i = 0; i < 3; i++){
        const float fs = init[9], ts = i == 2 ? init[11] / 100 : init[11];
        force[i] = fs == 0 ? init[8] : nrm[i] * fs + init[8];
        torque[i] = ts == 0 ? init[10] : nrm[3 + i] * ts + init[10];
    }
    float min_rpm, max_rpm;
    if(init[5] != 0.0f){
        min_rpm = (init[6] + 1) / 2 * (action_max - action_min) + action_min;
        max_rpm = (init[7] + 1) / 2 * (action_max - action_min) + action_min;
    }
    else{
        min_rpm = init[6] < 0 ? action_min : init[6];
        max_rpm = init[7] < 0 ? action_max : init[7];
        if(max_rpm > action_max) max_rpm = action_max;
        if(min_rpm > max_rpm) min_rpm = max_rpm;
    }
    for(int i = 0; i < 4; i++) rpm[i] = u[13 + i] * (max_rpm - min_rpm) + min_rpm;
}
/* the standard normal under orc_normal (Marsaglia polar on canonical draws, second value discarded) */
static float orc_standard_normal(orc_rng* r){
    float x, y, r2;
    do{
        x = 2.0f * orc_canonical(r) - 1.0f;
        y = 2.0f * orc_canonical(r) - 1.0f;
        r2 = x * x + y * y;
    } while(r2 > 1.0f || r2 == 0.0f);
    return y * sqrtf(-2 * logf(r2) / r2);
}
/* n x sample_initial_state on ONE engine, consuming it exactly where the reference does: no position / orientation / velocity draws under    */
/* guidance, no orientation draws for max_angle <= 0, no draw for a normal with std == 0. states [n, 23].                                    */
void orc_l2f_sample_initial_states(uint32_t seed, int n, const float* init, float action_min, float action_max, float* states){
    orc_rng r; orc_rng_init(&r, seed);
    for(int e = 0; e < n; e++){
        float u[17] = {0}, nrm[6] = {0};
        u[0] = orc_canonical(&r);
        const int guidance = u[0] < init[0];
        if(!guidance) for(int i = 0; i < 3; i++) u[1 + i] = orc_canonical(&r);
        if(init[2] > 0 && !guidance) for(int i = 0; i < 3; i++) u[4 + i] = orc_canonical(&r);
        if(!guidance) for(int i = 0; i < 6; i++) u[7 + i] = orc_canonical(&r);
        for(int i = 0; i < 3; i++) if(init[9] != 0) nrm[i] = orc_standard_normal(&r);
        for(int i = 0; i < 3; i++) if((i == 2 ? init[11] / 100 : init[11]) != 0) nrm[3 + i] = orc_standard_normal(&r);
        for(int i = 0; i < 4; i++) u[13 + i] = orc_canonical(&r);
        orc_l2f_initial_state_from_draws(init, action_min, action_max, u, nrm, states + (size_t)e * 23);
    }
}
