// What a layer does to a raw score q . k * scale before it weighs a key, and how the weights of a
// query's keys are formed.  All of it is float32.
//
//   s <- cap * tanh(s / cap)                      if cap > 0
//   s <- s - r1[head] * ln(1 + r2[head] * (i - j))   if r1 is given (i the query's position, j the key's)
//   weighting 0: softmax over the visible keys
//             1: softmax with one more term exp(0) in the denominator that carries no value
//             2: each visible key weighs sigmoid(s + head_bias[head]); nothing is normalised over keys
#pragma once
#include <math.h>

#define KESTREL_WEIGH_SOFTMAX 0
#define KESTREL_WEIGH_SOFTMAX_SINK 1
#define KESTREL_WEIGH_SIGMOID 2

struct ScoreOpts {
    float softcap;             // 0: none
    const float *r1, *r2;      // [nq] each, or both null
    const float *head_bias;    // [nq] or null; read by weighting 2 only
    int weighting;
};

// the options of one head, fetched once
struct HeadScore {
    float cap, inv_cap, r1, r2, bias;
    bool dist;
    __device__ __forceinline__ HeadScore(const ScoreOpts &o, int head) {
        cap = o.softcap;
        inv_cap = o.softcap > 0.f ? 1.0f / o.softcap : 0.f;
        dist = o.r1 != nullptr;
        r1 = dist ? o.r1[head] : 0.f;
        r2 = dist ? o.r2[head] : 0.f;
        bias = (o.weighting == KESTREL_WEIGH_SIGMOID && o.head_bias) ? o.head_bias[head] : 0.f;
    }
    // s = q . k * scale of a key `distance` positions behind the query
    __device__ __forceinline__ float operator()(float s, int distance) const {
        if (cap > 0.f) s = cap * tanhf(s * inv_cap);
        if (dist) s -= r1 * logf(1.0f + r2 * (float)distance);
        return s + bias;
    }
};

__device__ __forceinline__ float sigmoid_f32(float z) { return 1.0f / (1.0f + expf(-z)); }
