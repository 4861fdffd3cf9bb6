// A feed-forward of routed experts: the router's choice per token, and the experts' activation with the choice applied.
//
// Router: scores s = sigmoid(z) of the fp32 router logits z [tokens, E]. The E experts form `groups` equal groups of
// neighbours; a group's score is the sum of its two largest s (of its only one, when groups hold one expert); only experts
// of the `keep` best groups can be chosen. The `top` allowed experts with the largest s are chosen (the lower index wins a
// tie); their weights are their s divided by the sum of the chosen s (+ 1e-20), times `scale`. All of it in fp32.
//
// The choice leaves the kernel twice: as lists (expert ids and weights, [tokens, top]) and as a dense row per token
// (gate [tokens, E]: the weight of a chosen expert, 0 for the others). With the dense row the experts run as two
// products over ALL experts' stacked weights: u = h W_up^T [tokens, E ff], a = gate[expert of the column] act(u), and
// y = a W_down^T sums over experts inside the product's reduction; an expert that was not chosen adds exact zeros.
#include "common.cuh"

constexpr int ROUTE_MAX_TOP = 32;
constexpr int ROUTE_MAX_GROUPS = 64;

__global__ void route_kernel(float* __restrict__ gate, int* __restrict__ ids, float* __restrict__ wts, const float* __restrict__ z, int n_tokens,
                             int E, int top, int groups, int keep, float scale) {
    const int t = blockIdx.x * blockDim.x + threadIdx.x;
    if (t >= n_tokens) return;
    float* row = gate + (size_t)t * E;          // scratch for the scores until the last pass
    const float* zr = z + (size_t)t * E;
    for (int e = 0; e < E; ++e) row[e] = 1.f / (1.f + expf(-zr[e]));
    unsigned long long allowed = ~0ull;        // one bit per group
    const int per = E / groups;
    if (groups > 1 && keep < groups) {
        float score[ROUTE_MAX_GROUPS];
        for (int g = 0; g < groups; ++g) {
            float a = -1.f, b = -1.f;           // the two largest of the group (scores are >= 0)
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = row[e];
                if (v > a) { b = a; a = v; }
                else if (v > b) b = v;
            }
            score[g] = a + (b >= 0.f ? b : 0.f);
        }
        allowed = 0ull;
        for (int i = 0; i < keep; ++i) {
            int best = -1;
            float best_v = -INFINITY;
            for (int g = 0; g < groups; ++g)
                if (!((allowed >> g) & 1ull) && score[g] > best_v) { best_v = score[g]; best = g; }
            if (best >= 0) allowed |= 1ull << best;
        }
    }
    int chosen[ROUTE_MAX_TOP];
    float chosen_s[ROUTE_MAX_TOP];
    float sum = 0.f;
    for (int i = 0; i < top; ++i) {
        int best = -1;
        float best_v = -INFINITY;
        for (int e = 0; e < E; ++e) {
            const float v = row[e];             // -1 once chosen
            if (v >= 0.f && ((allowed >> (e / per)) & 1ull) && v > best_v) { best_v = v; best = e; }
        }
        chosen[i] = best;
        chosen_s[i] = best >= 0 ? best_v : 0.f;
        if (best >= 0) { row[best] = -1.f; sum += best_v; }
    }
    const float norm = scale / (sum + 1e-20f);
    for (int e = 0; e < E; ++e) row[e] = 0.f;
    for (int i = 0; i < top; ++i) {
        const float w = chosen_s[i] * norm;
        if (chosen[i] >= 0) row[chosen[i]] = w;
        ids[(size_t)t * top + i] = chosen[i];
        wts[(size_t)t * top + i] = w;
    }
}

OXR_API int oxr_route(float* gate, int* ids, float* wts, const float* z, int n_tokens, int E, int top, int groups, int keep, float scale,
                      cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || top <= 0 || top > E || top > ROUTE_MAX_TOP || groups <= 0 || groups > ROUTE_MAX_GROUPS || E % groups || keep <= 0 || keep > groups ||
        top > keep * (E / groups))
        return OXR_BAD_ARGUMENT;
    route_kernel<<<(n_tokens + 63) / 64, 64, 0, stream>>>(gate, ids, wts, z, n_tokens, E, top, groups, keep, scale);
    return oxr_launch_status();
}

// a[t, c] = gate[t, c / ff] * relu(u[t, c])^2 over the stacked columns of all experts; the product in fp32, rounded once.
template <typename T>
__global__ void gated_relu2_kernel(T* __restrict__ a, const T* __restrict__ u, const float* __restrict__ gate, size_t total, int cols, int ff, int E) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= total) return;
    const size_t t = i / cols;
    const int c = (int)(i - t * cols);
    const float g = gate[t * E + c / ff];
    const float v = fmaxf(Num<T>::to_f32(u[i]), 0.f);
    a[i] = Num<T>::from_f32(g * (v * v));
}

OXR_API int oxr_gated_relu2(void* a, const void* u, const float* gate, int n_tokens, int E, int ff, int dtype, cudaStream_t stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || ff <= 0) return OXR_BAD_ARGUMENT;
    const size_t total = (size_t)n_tokens * E * ff;
    const unsigned blocks = (unsigned)((total + 255) / 256);
    if (dtype == 0) gated_relu2_kernel<float><<<blocks, 256, 0, stream>>>((float*)a, (const float*)u, gate, total, E * ff, ff, E);
    else gated_relu2_kernel<__nv_bfloat16><<<blocks, 256, 0, stream>>>((__nv_bfloat16*)a, (const __nv_bfloat16*)u, gate, total, E * ff, ff, E);
    return oxr_launch_status();
}
