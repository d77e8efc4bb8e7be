// TinyMLP host class over the C ABI.  Behaviour follows the reference class (modules/TinyMLP/TinyMLP.cu):
// power-of-two padding of all dims (minimum 8), U(-1/sqrt(fan_in), 1/sqrt(fan_in)) weights from std::mt19937(seed)
// with zero biases (:86-105), training-only methods throwing std::runtime_error in inference mode (:257-263,
// 321, 355-393), Adam bias correction with the step counter capped at 50000 (:392-400), the raw-struct weight
// file format (:406-481).
#include "TinyMLP.h"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <random>

#include "host_kernels.h"

namespace nb {

void throw_on_error(int status, const char* what) {
    if (status != NB_OK) throw std::runtime_error(std::string(what) + ": " + nb_last_error());
}

void throw_on_cuda(cudaError_t e, const char* what) {
    if (e != cudaSuccess) throw std::runtime_error(std::string(what) + ": " + cudaGetErrorString(e));
}

void DeviceMem::allocate(size_t bytes, bool zero) {
    release();
    if (bytes == 0) return;
    throw_on_cuda(cudaMalloc(&ptr_, bytes), "cudaMalloc");
    bytes_ = bytes;
    if (zero) throw_on_cuda(cudaMemset(ptr_, 0, bytes), "cudaMemset");
}

void DeviceMem::adopt(void* ptr, size_t bytes) {
    release();
    ptr_ = ptr;
    bytes_ = ptr ? bytes : 0;
    owned_ = false;
}

void DeviceMem::release() {
    if (ptr_ && owned_) cudaFree(ptr_);
    ptr_ = nullptr;
    bytes_ = 0;
    owned_ = true;
}

void ParamArena::allocate(int64_t total_elems, int64_t sparse_elems, bool with_training) {
    total = (total_elems + 3) / 4 * 4;
    sparse_count = sparse_elems;
    w.allocate((size_t)total * sizeof(float), true);
    w_h.allocate((size_t)total * sizeof(half), true);
    training = false;
    if (with_training) enable_training();
}

void ParamArena::set_external_grad(float* ptr) {
    external_grad = ptr;
    if (!training) return;
    g.release();
    if (ptr) {
        g.adopt(ptr, (size_t)total * sizeof(float));
        throw_on_cuda(cudaMemset(ptr, 0, (size_t)total * sizeof(float)), "cudaMemset");
    } else {
        g.allocate((size_t)total * sizeof(float), true);
    }
}

void ParamArena::enable_training() {
    if (!g && external_grad) {
        g.adopt(external_grad, (size_t)total * sizeof(float));
        throw_on_cuda(cudaMemset(external_grad, 0, (size_t)total * sizeof(float)), "cudaMemset");
    }
    if (!g) g.allocate((size_t)total * sizeof(float), true);
    if (!m) m.allocate((size_t)total * sizeof(float), true);
    if (!v) v.allocate((size_t)total * sizeof(float), true);
    training = true;
}

void ParamArena::disable_training() {
    g.release(); m.release(); v.release();
    training = false;
}

void ParamArena::upload(int64_t off, const float* host, int64_t count) {
    if (count <= 0) return;
    std::vector<half> hh((size_t)count);
    for (int64_t i = 0; i < count; i++) hh[(size_t)i] = __float2half(host[i]);  // round to nearest even, as __float2half on the device
    throw_on_cuda(cudaMemcpy(W(off), host, (size_t)count * sizeof(float), cudaMemcpyHostToDevice), "upload parameters");
    throw_on_cuda(cudaMemcpy(Wh(off), hh.data(), (size_t)count * sizeof(half), cudaMemcpyHostToDevice), "upload fp16 parameters");
}

void ParamArena::download(int64_t off, float* host, int64_t count) const {
    if (count <= 0) return;
    throw_on_cuda(cudaMemcpy(host, W(off), (size_t)count * sizeof(float), cudaMemcpyDeviceToHost), "download parameters");
}

}  // namespace nb

static inline int layer_in(const MLPOption& o, int l) { return l == 0 ? o.inputDim : o.hiddenDim; }
static inline int layer_out(const MLPOption& o, int l) { return l == o.numLayers - 1 ? o.outputDim : o.hiddenDim; }

static MLPOption padded(const MLPOption& u) {
    MLPOption h = u;
    h.inputDim = nb::next_pow2_min8(u.inputDim);
    h.hiddenDim = nb::next_pow2_min8(u.hiddenDim);
    h.outputDim = nb::next_pow2_min8(u.outputDim);
    return h;
}

int64_t TinyMLP::paramCount(const MLPOption& options) {
    MLPOption h = padded(options);
    int64_t c = 0;
    for (int l = 0; l < h.numLayers; l++) c += (int64_t)layer_in(h, l) * layer_out(h, l) + layer_out(h, l);
    return c;
}

TinyMLP::TinyMLP(const MLPOption& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining)
    : TinyMLP(options, maxBatchSize, inferBatchSize, seed, isTraining, nullptr, 0) {}

TinyMLP::TinyMLP(const MLPOption& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining, nb::ParamArena* arena,
                 int64_t arena_offset)
    : user_opt(options), hw_opt(padded(options)), m_maxBatchSize(maxBatchSize),
      m_inferBatchSize(inferBatchSize <= 0 ? maxBatchSize : inferBatchSize), m_isTraining(isTraining) {
    if (options.numLayers < 1 || options.numLayers > NB_MAX_LAYERS) throw std::runtime_error("TinyMLP: numLayers must be between 1 and 8");
    desc_.input_dim = hw_opt.inputDim; desc_.hidden_dim = hw_opt.hiddenDim; desc_.output_dim = hw_opt.outputDim;
    desc_.num_layers = hw_opt.numLayers; desc_.output_activation = hw_opt.outputActivation;
    for (int l = 0; l < hw_opt.numLayers; l++) {
        n_w_ += (int64_t)layer_in(hw_opt, l) * layer_out(hw_opt, l);
        n_b_ += layer_out(hw_opt, l);
    }
    if (arena == nullptr) {
        owned_.reset(new nb::ParamArena());
        owned_->allocate(n_w_ + n_b_, 0, isTraining);
        arena_ = owned_.get();
        off_w_ = 0;
    } else {
        if (arena_offset % 8 != 0 || arena_offset + n_w_ + n_b_ > arena->total) throw std::runtime_error("TinyMLP: arena slice out of range or misaligned");
        arena_ = arena;
        off_w_ = arena_offset;
    }
    off_b_ = off_w_ + n_w_;
    allocate_buffers();
    init(seed);
}

TinyMLP::~TinyMLP() = default;

void TinyMLP::init(unsigned int seed) {
    std::mt19937 gen(seed);
    std::vector<float> w((size_t)n_w_), b((size_t)n_b_, 0.0f);
    size_t k = 0;
    for (int l = 0; l < hw_opt.numLayers; l++) {
        int in_d = layer_in(hw_opt, l), out_d = layer_out(hw_opt, l);
        float bound = 1.0f / std::sqrt((float)in_d);
        std::uniform_real_distribution<float> dist(-bound, bound);
        for (int i = 0; i < in_d * out_d; i++) w[k++] = dist(gen);
    }
    arena_->upload(off_w_, w.data(), n_w_);
    arena_->upload(off_b_, b.data(), n_b_);
}

void TinyMLP::allocate_buffers() {
    size_t max_pad = (size_t)std::max(m_maxBatchSize, m_inferBatchSize);
    bool needs_in_pad = user_opt.inputDim != hw_opt.inputDim;
    bool needs_out_pad = user_opt.outputDim != hw_opt.outputDim;
    if ((m_isTraining || needs_in_pad) && !padded_in_) padded_in_.allocate(max_pad * hw_opt.inputDim * sizeof(half));
    if ((m_isTraining || needs_out_pad) && !padded_out_) padded_out_.allocate(max_pad * hw_opt.outputDim * sizeof(float));
    if (m_isTraining) {
        size_t mb = (size_t)m_maxBatchSize;
        if (!padded_targets_) padded_targets_.allocate(mb * hw_opt.outputDim * sizeof(half));
        if (!dloss_) dloss_.allocate(mb * hw_opt.outputDim * sizeof(half));
        if (!total_loss_) total_loss_.allocate(sizeof(float), true);
        if (!acts_ && hw_opt.numLayers > 1) acts_.allocate(mb * hw_opt.hiddenDim * sizeof(half) * (hw_opt.numLayers - 1));
        if (owned_) owned_->enable_training();
    }
}

void TinyMLP::switchToInferenceMode() {
    if (!m_isTraining) return;
    if (user_opt.inputDim == hw_opt.inputDim) padded_in_.release();
    if (user_opt.outputDim == hw_opt.outputDim) padded_out_.release();
    padded_targets_.release(); dloss_.release(); total_loss_.release(); acts_.release();
    if (owned_) owned_->disable_training();
    m_isTraining = false;
}

void TinyMLP::switchToTrainingMode() {
    if (m_isTraining) return;
    m_isTraining = true;
    allocate_buffers();
}

void TinyMLP::zero_grad(cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("zero_grad called while in inference mode!");
    nb::throw_on_error(nb_zero_async(arena_->G(off_w_), (n_w_ + n_b_) * (int64_t)sizeof(float), stream), "zero_grad");
}

void TinyMLP::forward(const half* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("forward called while in inference mode!");
    if (batchSize > m_maxBatchSize) throw std::runtime_error("Batch size exceeds maxBatchSize");
    if (user_opt.inputDim != hw_opt.inputDim) {
        nb::pad_rows_half(d_unpadded_inputs, padded_in_.as<half>(), batchSize, user_opt.inputDim, hw_opt.inputDim, stream);
    } else {
        // the layer-0 input is snapshotted: backward reads it after the caller may have reused its buffer
        nb::throw_on_cuda(cudaMemcpyAsync(padded_in_.as<half>(), d_unpadded_inputs, (size_t)batchSize * hw_opt.inputDim * sizeof(half),
                                          cudaMemcpyDeviceToDevice, stream), "forward: input snapshot");
    }
    nb::throw_on_error(nb_mlp_forward(&desc_, padded_in_.as<half>(), arena_->Wh(off_w_), arena_->W(off_b_), batchSize, padded_out_.as<float>(),
                                      acts_.as<half>(), stream), "TinyMLP::forward");
    if (d_outputs != nullptr) {
        if (user_opt.outputDim == hw_opt.outputDim)
            nb::throw_on_cuda(cudaMemcpyAsync(d_outputs, padded_out_.as<float>(), (size_t)batchSize * hw_opt.outputDim * sizeof(float),
                                              cudaMemcpyDeviceToDevice, stream), "forward: output copy");
        else
            nb::unpad_rows_float(padded_out_.as<float>(), d_outputs, batchSize, hw_opt.outputDim, user_opt.outputDim, stream);
    }
}

void TinyMLP::inference(const half* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream) {
    if (batchSize > m_inferBatchSize) {
        for (int offset = 0; offset < batchSize; offset += m_inferBatchSize) {
            int cur = std::min(m_inferBatchSize, batchSize - offset);
            inference(d_unpadded_inputs + (size_t)offset * user_opt.inputDim,
                      d_outputs ? d_outputs + (size_t)offset * user_opt.outputDim : nullptr, cur, stream);
        }
        return;
    }
    const half* in = d_unpadded_inputs;
    if (user_opt.inputDim != hw_opt.inputDim) {
        nb::pad_rows_half(d_unpadded_inputs, padded_in_.as<half>(), batchSize, user_opt.inputDim, hw_opt.inputDim, stream);
        in = padded_in_.as<half>();
    }
    if (user_opt.outputDim == hw_opt.outputDim) {
        if (d_outputs == nullptr) return;  // nowhere to write (the reference launches into a null pointer here)
        nb::throw_on_error(nb_mlp_forward(&desc_, in, arena_->Wh(off_w_), arena_->W(off_b_), batchSize, d_outputs, nullptr, stream),
                           "TinyMLP::inference");
    } else {
        nb::throw_on_error(nb_mlp_forward(&desc_, in, arena_->Wh(off_w_), arena_->W(off_b_), batchSize, padded_out_.as<float>(), nullptr, stream),
                           "TinyMLP::inference");
        if (d_outputs != nullptr) nb::unpad_rows_float(padded_out_.as<float>(), d_outputs, batchSize, hw_opt.outputDim, user_opt.outputDim, stream);
    }
}

float TinyMLP::calculate_loss_and_grad(const half* d_unpadded_targets, int batchSize, float loss_scale, bool fetch_loss, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("calculate_loss_and_grad called while in inference mode!");
    nb::throw_on_error(nb_zero_async(total_loss_.as<float>(), sizeof(float), stream), "loss reset");
    const half* targets = d_unpadded_targets;
    if (user_opt.outputDim != hw_opt.outputDim) {
        nb::pad_rows_half(d_unpadded_targets, padded_targets_.as<half>(), batchSize, user_opt.outputDim, hw_opt.outputDim, stream);
        targets = padded_targets_.as<half>();
    }
    nb::throw_on_error(nb_mse_loss_grad(padded_out_.as<float>(), targets, dloss_.as<half>(), total_loss_.as<float>(), batchSize, hw_opt.outputDim,
                                        user_opt.outputDim, loss_scale, hw_opt.outputActivation, stream), "calculate_loss_and_grad");
    if (fetch_loss) {
        float h_loss = 0.f;
        nb::throw_on_cuda(cudaMemcpyAsync(&h_loss, total_loss_.as<float>(), sizeof(float), cudaMemcpyDeviceToHost, stream), "loss fetch");
        nb::throw_on_cuda(cudaStreamSynchronize(stream), "loss fetch");
        return h_loss / (batchSize * user_opt.outputDim);
    }
    return 0.0f;
}

const half* TinyMLP::stage_grad(const half* custom_loss_grad, int batchSize, cudaStream_t stream) {
    if (user_opt.outputDim != hw_opt.outputDim) {
        nb::pad_rows_half(custom_loss_grad, dloss_.as<half>(), batchSize, user_opt.outputDim, hw_opt.outputDim, stream);
        return dloss_.as<half>();
    }
    return custom_loss_grad;  // already in the kernel's layout: consumed in place (the reference copies it first)
}

void TinyMLP::run_backward(const half* grad_padded, half* dx_out, int batchSize, cudaStream_t stream) {
    nb::throw_on_error(nb_mlp_backward(&desc_, grad_padded, arena_->Wh(off_w_), padded_in_.as<half>(), acts_.as<half>(), batchSize,
                                       arena_->G(off_w_), arena_->G(off_b_), dx_out, stream), "TinyMLP::backward");
}

void TinyMLP::backward(int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    run_backward(dloss_.as<half>(), nullptr, batchSize, stream);
}

void TinyMLP::backward(const half* custom_loss_grad, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    run_backward(stage_grad(custom_loss_grad, batchSize, stream), nullptr, batchSize, stream);
}

void TinyMLP::backward(half* out_d_dx_out, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    run_backward(dloss_.as<half>(), out_d_dx_out, batchSize, stream);
}

void TinyMLP::backward(const half* custom_loss_grad, half* out_d_dx_out, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    run_backward(stage_grad(custom_loss_grad, batchSize, stream), out_d_dx_out, batchSize, stream);
}

void TinyMLP::reset_step() { current_step = 0; }

void TinyMLP::step(float lr, float beta1, float beta2, float epsilon, float loss_scale, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("step called while in inference mode!");
    if (current_step < 50000) current_step++;
    float bc1 = 1.0f - std::pow(beta1, (float)current_step);
    float bc2 = 1.0f - std::pow(beta2, (float)current_step);
    nb::throw_on_error(nb_adam_step(arena_->W(off_w_), arena_->Wh(off_w_), arena_->G(off_w_), arena_->M(off_w_), arena_->V(off_w_), 0,
                                    n_w_ + n_b_, lr, beta1, beta2, epsilon, bc1, bc2, 1.0f / loss_scale, 0, stream), "TinyMLP::step");
}

void TinyMLP::loadWeights(const std::string& filename) {
    std::ifstream in(filename, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Cannot open file for loading weights: " + filename);
    MLPOption file_opt;
    in.read(reinterpret_cast<char*>(&file_opt), sizeof(MLPOption));
    if (file_opt.inputDim != hw_opt.inputDim || file_opt.hiddenDim != hw_opt.hiddenDim || file_opt.outputDim != hw_opt.outputDim ||
        file_opt.numLayers != hw_opt.numLayers)
        throw std::runtime_error("Weight file dimension mismatch!");
    std::vector<float> w((size_t)n_w_), b((size_t)n_b_);
    size_t wo = 0, bo = 0;
    for (int l = 0; l < hw_opt.numLayers; l++) {  // the file interleaves W_l, b_l per layer
        size_t we = (size_t)layer_in(hw_opt, l) * layer_out(hw_opt, l), be = (size_t)layer_out(hw_opt, l);
        in.read(reinterpret_cast<char*>(w.data() + wo), we * sizeof(float));
        in.read(reinterpret_cast<char*>(b.data() + bo), be * sizeof(float));
        wo += we; bo += be;
    }
    if (!in) throw std::runtime_error("Weight file truncated: " + filename);
    loadWeights(w.data(), b.data());
}

void TinyMLP::saveWeights(const std::string& filename) {
    std::ofstream out(filename, std::ios::binary);
    if (!out.is_open()) throw std::runtime_error("Cannot open file for saving weights: " + filename);
    out.write(reinterpret_cast<const char*>(&hw_opt), sizeof(MLPOption));
    std::vector<float> w((size_t)n_w_), b((size_t)n_b_);
    saveWeights(w.data(), b.data());
    size_t wo = 0, bo = 0;
    for (int l = 0; l < hw_opt.numLayers; l++) {
        size_t we = (size_t)layer_in(hw_opt, l) * layer_out(hw_opt, l), be = (size_t)layer_out(hw_opt, l);
        out.write(reinterpret_cast<const char*>(w.data() + wo), we * sizeof(float));
        out.write(reinterpret_cast<const char*>(b.data() + bo), be * sizeof(float));
        wo += we; bo += be;
    }
}

void TinyMLP::loadWeights(const float* host_weights, const float* host_biases) {
    arena_->upload(off_w_, host_weights, n_w_);
    arena_->upload(off_b_, host_biases, n_b_);
}

void TinyMLP::saveWeights(float* host_weights, float* host_biases) {
    nb::throw_on_cuda(cudaDeviceSynchronize(), "saveWeights");
    arena_->download(off_w_, host_weights, n_w_);
    arena_->download(off_b_, host_biases, n_b_);
}
