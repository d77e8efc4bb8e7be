// Host class of the plain fused MLP, source-compatible with the reference's TinyMLP
// (modules/TinyMLP/TinyMLP.h:26-85): same option struct, constructor, methods, defaults and exceptions, so code
// written against the reference compiles against this header.  Underneath it drives the C ABI of
// include/nerf_b200.h; parameters, gradients and Adam moments live in one flat arena (optionally shared with
// other networks, see nb::ParamArena) instead of per-layer allocations.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

#include "../../include/nerf_b200.h"

#define ACT_RELU 0
#define OUT_ACT_NONE 0
#define OUT_ACT_SIGMOID 1

// Field order is part of the weight-file format (modules/TinyMLP/TinyMLP.h:26-33, TinyMLP.cu:452-456).
struct MLPOption {
    int inputDim;
    int hiddenDim;
    int outputDim;
    int numLayers;
    int activationType;
    int outputActivation = OUT_ACT_NONE;
};

namespace nb {

// Throws std::runtime_error carrying nb_last_error() when a C-ABI call fails.
void throw_on_error(int status, const char* what);
void throw_on_cuda(cudaError_t e, const char* what);

// RAII device allocation (non-copyable).
class DeviceMem {
public:
    DeviceMem() = default;
    ~DeviceMem() { release(); }
    DeviceMem(const DeviceMem&) = delete;
    DeviceMem& operator=(const DeviceMem&) = delete;
    void allocate(size_t bytes, bool zero = false);
    // Uses memory the caller owns (and keeps alive) instead of allocating; release() then only forgets it.
    void adopt(void* ptr, size_t bytes);
    void release();
    template <class T> T* as() const { return static_cast<T*>(ptr_); }
    size_t bytes() const { return bytes_; }
    explicit operator bool() const { return ptr_ != nullptr; }
private:
    void* ptr_ = nullptr;
    size_t bytes_ = 0;
    bool owned_ = true;
};

// One flat run of parameters with everything the optimizer needs, element i of every array describing the same
// parameter: fp32 master value, fp16 copy used by the forward kernels, fp32 gradient, Adam moments.
// Elements [0, sparse_count) are hash-table entries (sparse Adam rule), the rest dense network parameters.
struct ParamArena {
    int64_t total = 0;
    int64_t sparse_count = 0;
    DeviceMem w, w_h, g, m, v;
    bool training = false;
    void allocate(int64_t total_elems, int64_t sparse_elems, bool with_training);
    void enable_training();   // allocates g, m, v (zeroed) if missing
    // The gradient lives in caller-owned memory of at least `total` floats from now on (e.g. a buffer registered with a
    // collective library); it is zeroed here and used again whenever training is re-enabled.  nullptr returns to an
    // own allocation.
    void set_external_grad(float* ptr);
    float* external_grad = nullptr;
    void disable_training();  // frees g, m, v
    float* W(int64_t off = 0) const { return w.as<float>() + off; }
    half* Wh(int64_t off = 0) const { return w_h.as<half>() + off; }
    float* G(int64_t off = 0) const { return g.as<float>() + off; }
    float* M(int64_t off = 0) const { return m.as<float>() + off; }
    float* V(int64_t off = 0) const { return v.as<float>() + off; }
    // host fp32 -> master + fp16 copy
    void upload(int64_t off, const float* host, int64_t count);
    void download(int64_t off, float* host, int64_t count) const;
};

inline int next_pow2_min8(int n) {
    if (n <= 8) return 8;
    n--;
    n |= n >> 1; n |= n >> 2; n |= n >> 4; n |= n >> 8; n |= n >> 16;
    return n + 1;
}

}  // namespace nb

class TinyMLP {
public:
    explicit TinyMLP(const MLPOption& options, int maxBatchSize, int inferBatchSize = 0, unsigned int seed = 42, bool isTraining = true);
    // Places the network's parameters inside an existing arena at element offset `arena_offset` (weights of all
    // layers, then biases of all layers).  The arena must outlive the object.  No counterpart in the reference.
    TinyMLP(const MLPOption& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining, nb::ParamArena* arena,
            int64_t arena_offset);
    ~TinyMLP();
    TinyMLP(const TinyMLP&) = delete;
    TinyMLP& operator=(const TinyMLP&) = delete;

    void switchToInferenceMode();
    void switchToTrainingMode();

    void zero_grad(cudaStream_t stream = 0);
    void forward(const half* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream = 0);
    float calculate_loss_and_grad(const half* d_unpadded_targets, int batchSize, float loss_scale = 65536.0f, bool fetch_loss = false,
                                  cudaStream_t stream = 0);
    void backward(int batchSize, cudaStream_t stream = 0);
    void backward(const half* custom_loss_grad, int batchSize, cudaStream_t stream = 0);
    void backward(half* out_d_dx_out, int batchSize, cudaStream_t stream = 0);
    void backward(const half* custom_loss_grad, half* out_d_dx_out, int batchSize, cudaStream_t stream = 0);
    void step(float lr = 3e-4f, float beta1 = 0.9f, float beta2 = 0.999f, float epsilon = 1e-8f, float loss_scale = 65536.0f,
              cudaStream_t stream = 0);
    void reset_step();
    void inference(const half* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream = 0);

    void loadWeights(const std::string& filename);
    void saveWeights(const std::string& filename);
    void loadWeights(const float* host_weights, const float* host_biases);
    void saveWeights(float* host_weights, float* host_biases);

    // ---- additions (not in the reference) -------------------------------------------------------------
    static int64_t paramCount(const MLPOption& options);  // padded weights + biases, what the arena must hold
    const nb_mlp_desc& desc() const { return desc_; }
    int64_t weightOffset() const { return off_w_; }
    int64_t biasOffset() const { return off_b_; }
    int64_t weightCount() const { return n_w_; }
    int64_t biasCount() const { return n_b_; }
    bool isTraining() const { return m_isTraining; }
    // padded fp32 output of the last forward/inference ([batch][padded outputDim])
    float* paddedOutput() const { return padded_out_.as<float>(); }

private:
    void init(unsigned int seed);
    void allocate_buffers();
    void run_backward(const half* grad_padded, half* dx_out, int batchSize, cudaStream_t stream);
    const half* stage_grad(const half* custom_loss_grad, int batchSize, cudaStream_t stream);

    MLPOption user_opt;
    MLPOption hw_opt;
    nb_mlp_desc desc_{};
    int m_maxBatchSize;
    int m_inferBatchSize;
    int current_step = 0;
    bool m_isTraining;

    std::unique_ptr<nb::ParamArena> owned_;
    nb::ParamArena* arena_ = nullptr;
    int64_t off_w_ = 0, off_b_ = 0, n_w_ = 0, n_b_ = 0;

    nb::DeviceMem padded_in_, padded_targets_, padded_out_, dloss_, total_loss_, acts_;
};
