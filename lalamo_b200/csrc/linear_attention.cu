// Linear attention with a decaying matrix state per head and no softmax or denominator:
//
//   S_t = diag(a_t) S_(t-1) + k_t v_t^T,     o_t = S_t^T q_t
//
// The decay a_t is one fixed number per head, repeated over the head's key channels, or one number per head and key
// channel made from the token: a = sigmoid(z)^(1 / tau), z a projection of the token plus a bias.  This file holds the
// kernel that lays the recurrence's inputs out in 32-bit (q, k and v as the projection left them, one of q and k
// times key_dim^-1/2, and the decays); the recurrence itself is the scan of gated_delta.cu without its delta-rule
// correction, and the read-out (per-head RMS norm times a gate) is that file's output kernel.
#include "common.cuh"

namespace lb {

// grid (tokens), threads over channels.
//   proj [tokens, stride]: q (heads x dk) | k (heads x dk) | v (heads x dv) | ...
//   z [tokens, z_stride] (may be null): decay logits, heads x dk;  z_bias (may be null): heads x dk
//   fixed_decay (used when z is null): heads
template <typename T>
__global__ void linear_attention_prepare_kernel(const T* __restrict__ proj, int stride, const T* __restrict__ z, int z_stride,
                                                const float* __restrict__ z_bias, const float* __restrict__ fixed_decay, float inverse_tau,
                                                float q_scale, float k_scale, float* __restrict__ q_out, float* __restrict__ k_out,
                                                float* __restrict__ v_out, float* __restrict__ g_out, int heads, int dk, int dv) {
    const int token = blockIdx.x;
    const T* row = proj + static_cast<size_t>(token) * stride;
    const int key_width = heads * dk, value_width = heads * dv;
    for (int index = threadIdx.x; index < key_width; index += blockDim.x) {
        q_out[static_cast<size_t>(token) * key_width + index] = to_float(row[index]) * q_scale;
        k_out[static_cast<size_t>(token) * key_width + index] = to_float(row[key_width + index]) * k_scale;
        float decay;
        if (z != nullptr) {
            const float logit = to_float(z[static_cast<size_t>(token) * z_stride + index]) + (z_bias != nullptr ? z_bias[index] : 0.0f);
            // log sigmoid(x) = min(x, 0) - log(1 + exp(-|x|)), and sigmoid(x)^(1 / tau) = exp(log sigmoid(x) / tau)
            const float log_sigmoid = fminf(logit, 0.0f) - log1pf(expf(-fabsf(logit)));
            decay = expf(log_sigmoid * inverse_tau);
        } else {
            decay = fixed_decay[index / dk];
        }
        g_out[static_cast<size_t>(token) * key_width + index] = decay;
    }
    for (int index = threadIdx.x; index < value_width; index += blockDim.x)
        v_out[static_cast<size_t>(token) * value_width + index] = to_float(row[2 * key_width + index]);
}

}  // namespace lb

extern "C" {

int lb_linear_attention_prepare(const void* proj, int stride, const void* z, int z_stride, const float* z_bias, const float* fixed_decay, float inverse_tau,
                                float q_scale, float k_scale, float* q_out, float* k_out, float* v_out, float* g_out, int tokens, int heads, int dk, int dv,
                                int dtype, cudaStream_t stream) {
    if (tokens == 0) return 0;
    if (z == nullptr && fixed_decay == nullptr) return -2;
    LB_DISPATCH_DTYPE(dtype, {
        lb::linear_attention_prepare_kernel<T><<<tokens, 256, 0, stream>>>(static_cast<const T*>(proj), stride, static_cast<const T*>(z), z_stride, z_bias,
                                                                            fixed_decay, inverse_tau, q_scale, k_scale, q_out, k_out, v_out, g_out, heads, dk, dv);
    })
    return LB_LAUNCH_RESULT();
}

}  // extern "C"
