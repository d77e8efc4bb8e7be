// TinyMLPHashGrid host class over the C ABI.  Behaviour follows the reference class
// (modules/TinyMLP/TinyMLPHashGrid.cu): vectorDim 3 or 4 and featuresLevel 2 enforced (:38-39), hidden and output
// dims padded to powers of two (:41-43), hash table U(-0.1, 0.1) then weights U(+-1/sqrt(fan_in)) from one
// std::mt19937(seed) (:55-82), the caller's float4 input pointer kept until backward when vectorDim == 4 (:258),
// file format = raw MLPGridOptions + fp32 table + per-layer W, b (:394-455).
#include "TinyMLPHashGrid.h"

#include <algorithm>
#include <cmath>
#include <fstream>
#include <random>

#include "host_kernels.h"

static inline int g_in(const MLPOption& o, int l) { return l == 0 ? o.inputDim : o.hiddenDim; }
static inline int g_out(const MLPOption& o, int l) { return l == o.numLayers - 1 ? o.outputDim : o.hiddenDim; }

int64_t TinyMLPHashGrid::mlpParamCount(const MLPGridOptions& o) {
    MLPOption m{o.numLevels * o.featuresLevel, nb::next_pow2_min8(o.hiddenDim), nb::next_pow2_min8(o.outputDim), o.numLayers, o.activationType};
    int64_t c = 0;
    for (int l = 0; l < m.numLayers; l++) c += (int64_t)g_in(m, l) * g_out(m, l) + g_out(m, l);
    return c;
}

TinyMLPHashGrid::TinyMLPHashGrid(const MLPGridOptions& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining)
    : user_opt(options), m_maxBatchSize(maxBatchSize), m_inferBatchSize(inferBatchSize <= 0 ? maxBatchSize : inferBatchSize),
      m_isTraining(isTraining) {
    construct(seed, nullptr, 0, 0);
}

TinyMLPHashGrid::TinyMLPHashGrid(const MLPGridOptions& options, int maxBatchSize, int inferBatchSize, unsigned int seed, bool isTraining,
                                 nb::ParamArena* arena, int64_t hash_offset, int64_t mlp_offset)
    : user_opt(options), m_maxBatchSize(maxBatchSize), m_inferBatchSize(inferBatchSize <= 0 ? maxBatchSize : inferBatchSize),
      m_isTraining(isTraining) {
    construct(seed, arena, hash_offset, mlp_offset);
}

TinyMLPHashGrid::~TinyMLPHashGrid() = default;

void TinyMLPHashGrid::construct(unsigned int seed, nb::ParamArena* arena, int64_t hash_offset, int64_t mlp_offset) {
    const MLPGridOptions& options = user_opt;
    if (options.vectorDim != 3 && options.vectorDim != 4) throw std::runtime_error("TinyMLPHashGrid: vectorDim must be 3 or 4");
    if (options.featuresLevel != 2) throw std::runtime_error("TinyMLPHashGrid: featuresLevel must be 2");
    if (options.numLayers < 1 || options.numLayers > NB_MAX_LAYERS) throw std::runtime_error("TinyMLPHashGrid: numLayers must be between 1 and 8");
    hw_opt = options;
    hw_opt.hiddenDim = nb::next_pow2_min8(options.hiddenDim);
    hw_opt.outputDim = nb::next_pow2_min8(options.outputDim);
    mlp_opt.inputDim = hw_opt.numLevels * hw_opt.featuresLevel;
    mlp_opt.hiddenDim = hw_opt.hiddenDim;
    mlp_opt.outputDim = hw_opt.outputDim;
    mlp_opt.numLayers = hw_opt.numLayers;
    mlp_opt.activationType = hw_opt.activationType;
    desc_.input_dim = mlp_opt.inputDim; desc_.hidden_dim = mlp_opt.hiddenDim; desc_.output_dim = mlp_opt.outputDim;
    desc_.num_layers = mlp_opt.numLayers; desc_.output_activation = 0;
    nb::throw_on_error(nb_grid_setup(&grid_, hw_opt.numLevels, hw_opt.tableSize, hw_opt.lowestSize, hw_opt.b, 0), "TinyMLPHashGrid: grid set-up");

    n_hash_ = hashCount(hw_opt);
    for (int l = 0; l < mlp_opt.numLayers; l++) {
        n_w_ += (int64_t)g_in(mlp_opt, l) * g_out(mlp_opt, l);
        n_b_ += g_out(mlp_opt, l);
    }
    if (arena == nullptr) {
        owned_.reset(new nb::ParamArena());
        owned_->allocate(n_hash_ + n_w_ + n_b_, n_hash_, m_isTraining);
        arena_ = owned_.get();
        off_hash_ = 0;
        off_w_ = n_hash_;
    } else {
        if (hash_offset % 8 || mlp_offset % 8 || hash_offset + n_hash_ > arena->total || mlp_offset + n_w_ + n_b_ > arena->total)
            throw std::runtime_error("TinyMLPHashGrid: arena slice out of range or misaligned");
        arena_ = arena;
        off_hash_ = hash_offset;
        off_w_ = mlp_offset;
    }
    off_b_ = off_w_ + n_w_;
    allocate_buffers();

    std::mt19937 gen(seed);
    {
        std::uniform_real_distribution<float> hash_dist(-0.1f, 0.1f);
        std::vector<float> h((size_t)n_hash_);
        for (auto& x : h) x = hash_dist(gen);
        arena_->upload(off_hash_, h.data(), n_hash_);
    }
    std::vector<float> w((size_t)n_w_), b((size_t)n_b_, 0.0f);
    size_t k = 0;
    for (int l = 0; l < mlp_opt.numLayers; l++) {
        int in_d = g_in(mlp_opt, l), out_d = g_out(mlp_opt, l);
        float bound = 1.0f / std::sqrt((float)in_d);
        std::uniform_real_distribution<float> w_dist(-bound, bound);
        for (int i = 0; i < in_d * out_d; i++) w[k++] = w_dist(gen);
    }
    arena_->upload(off_w_, w.data(), n_w_);
    arena_->upload(off_b_, b.data(), n_b_);
}

void TinyMLPHashGrid::allocate_buffers() {
    size_t max_pad = (size_t)std::max(m_maxBatchSize, m_inferBatchSize);
    bool needs_in_pad = user_opt.vectorDim != 4;
    bool needs_out_pad = user_opt.outputDim != hw_opt.outputDim;
    if (needs_in_pad && !padded_in_) padded_in_.allocate(max_pad * 4 * sizeof(float));
    if ((m_isTraining || needs_out_pad) && !padded_out_) padded_out_.allocate(max_pad * hw_opt.outputDim * sizeof(float));
    if (m_isTraining) {
        size_t mb = (size_t)m_maxBatchSize;
        if (!padded_targets_) padded_targets_.allocate(mb * hw_opt.outputDim * sizeof(half));
        if (!dloss_) dloss_.allocate(mb * hw_opt.outputDim * sizeof(half));
        if (!total_loss_) total_loss_.allocate(sizeof(float), true);
        if (!enc_) enc_.allocate(mb * mlp_opt.inputDim * sizeof(half));
        if (!denc_) denc_.allocate(mb * mlp_opt.inputDim * sizeof(half));
        if (!acts_ && mlp_opt.numLayers > 1) acts_.allocate(mb * mlp_opt.hiddenDim * sizeof(half) * (mlp_opt.numLayers - 1));
        if (owned_) owned_->enable_training();
    }
}

void TinyMLPHashGrid::switchToInferenceMode() {
    if (!m_isTraining) return;
    if (user_opt.outputDim == hw_opt.outputDim) padded_out_.release();
    padded_targets_.release(); dloss_.release(); total_loss_.release(); enc_.release(); denc_.release(); acts_.release();
    if (owned_) owned_->disable_training();
    m_isTraining = false;
}

void TinyMLPHashGrid::switchToTrainingMode() {
    if (m_isTraining) return;
    m_isTraining = true;
    allocate_buffers();
}

void TinyMLPHashGrid::zero_grad(cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("zero_grad called while in inference mode!");
    // only the network part: the hash-table gradient is zeroed by the optimizer as it consumes it
    nb::throw_on_error(nb_zero_async(arena_->G(off_w_), (n_w_ + n_b_) * (int64_t)sizeof(float), stream), "zero_grad");
}

void TinyMLPHashGrid::forward(const float* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("forward called while in inference mode!");
    if (batchSize > m_maxBatchSize) throw std::runtime_error("batchSize exceeds maxBatchSize");
    const float* in = d_unpadded_inputs;
    if (user_opt.vectorDim == 3) {
        nb::pad_rows_float(d_unpadded_inputs, padded_in_.as<float>(), batchSize, 3, 4, stream);
        in = padded_in_.as<float>();
    }
    last_inputs_ = in;
    nb::throw_on_error(nb_grid_mlp_forward(&grid_, &desc_, in, arena_->Wh(off_hash_), arena_->Wh(off_w_), arena_->W(off_b_), batchSize,
                                           padded_out_.as<float>(), enc_.as<half>(), acts_.as<half>(), stream), "TinyMLPHashGrid::forward");
    if (d_outputs != nullptr) {
        if (user_opt.outputDim == hw_opt.outputDim)
            nb::throw_on_cuda(cudaMemcpyAsync(d_outputs, padded_out_.as<float>(), (size_t)batchSize * hw_opt.outputDim * sizeof(float),
                                              cudaMemcpyDeviceToDevice, stream), "forward: output copy");
        else
            nb::unpad_rows_float(padded_out_.as<float>(), d_outputs, batchSize, hw_opt.outputDim, user_opt.outputDim, stream);
    }
}

void TinyMLPHashGrid::inference(const float* d_unpadded_inputs, float* d_outputs, int batchSize, cudaStream_t stream) {
    if (batchSize > m_inferBatchSize) {
        for (int offset = 0; offset < batchSize; offset += m_inferBatchSize) {
            int cur = std::min(m_inferBatchSize, batchSize - offset);
            inference(d_unpadded_inputs + (size_t)offset * user_opt.vectorDim,
                      d_outputs ? d_outputs + (size_t)offset * user_opt.outputDim : nullptr, cur, stream);
        }
        return;
    }
    const float* in = d_unpadded_inputs;
    if (user_opt.vectorDim == 3) {
        nb::pad_rows_float(d_unpadded_inputs, padded_in_.as<float>(), batchSize, 3, 4, stream);
        in = padded_in_.as<float>();
    }
    if (user_opt.outputDim == hw_opt.outputDim) {
        if (d_outputs == nullptr) return;
        nb::throw_on_error(nb_grid_mlp_forward(&grid_, &desc_, in, arena_->Wh(off_hash_), arena_->Wh(off_w_), arena_->W(off_b_), batchSize, d_outputs,
                                               nullptr, nullptr, stream), "TinyMLPHashGrid::inference");
    } else {
        nb::throw_on_error(nb_grid_mlp_forward(&grid_, &desc_, in, arena_->Wh(off_hash_), arena_->Wh(off_w_), arena_->W(off_b_), batchSize,
                                               padded_out_.as<float>(), nullptr, nullptr, stream), "TinyMLPHashGrid::inference");
        if (d_outputs != nullptr) nb::unpad_rows_float(padded_out_.as<float>(), d_outputs, batchSize, hw_opt.outputDim, user_opt.outputDim, stream);
    }
}

float TinyMLPHashGrid::calculate_loss_and_grad(const half* d_unpadded_targets, int batchSize, float loss_scale, bool fetch_loss,
                                               cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("calculate_loss_and_grad called while in inference mode!");
    nb::throw_on_error(nb_zero_async(total_loss_.as<float>(), sizeof(float), stream), "loss reset");
    const half* targets = d_unpadded_targets;
    if (user_opt.outputDim != hw_opt.outputDim) {
        nb::pad_rows_half(d_unpadded_targets, padded_targets_.as<half>(), batchSize, user_opt.outputDim, hw_opt.outputDim, stream);
        targets = padded_targets_.as<half>();
    }
    nb::throw_on_error(nb_mse_loss_grad(padded_out_.as<float>(), targets, dloss_.as<half>(), total_loss_.as<float>(), batchSize, hw_opt.outputDim,
                                        user_opt.outputDim, loss_scale, 0, stream), "calculate_loss_and_grad");
    if (fetch_loss) {
        float h_loss = 0.f;
        nb::throw_on_cuda(cudaMemcpyAsync(&h_loss, total_loss_.as<float>(), sizeof(float), cudaMemcpyDeviceToHost, stream), "loss fetch");
        nb::throw_on_cuda(cudaStreamSynchronize(stream), "loss fetch");
        return h_loss / (batchSize * user_opt.outputDim);
    }
    return 0.0f;
}

void TinyMLPHashGrid::run_backward(const half* grad_padded, int batchSize, cudaStream_t stream) {
    if (last_inputs_ == nullptr) throw std::runtime_error("backward called before forward");
    nb::throw_on_error(nb_mlp_backward(&desc_, grad_padded, arena_->Wh(off_w_), enc_.as<half>(), acts_.as<half>(), batchSize, arena_->G(off_w_),
                                       arena_->G(off_b_), denc_.as<half>(), stream), "TinyMLPHashGrid::backward (network)");
    nb::throw_on_error(nb_hash_scatter_backward(&grid_, last_inputs_, denc_.as<half>(), batchSize, arena_->G(off_hash_), stream),
                       "TinyMLPHashGrid::backward (scatter)");
}

void TinyMLPHashGrid::backward(int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    run_backward(dloss_.as<half>(), batchSize, stream);
}

void TinyMLPHashGrid::backward(const half* custom_loss_grad, int batchSize, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("backward called while in inference mode!");
    const half* g = custom_loss_grad;
    if (user_opt.outputDim != hw_opt.outputDim) {
        nb::pad_rows_half(custom_loss_grad, dloss_.as<half>(), batchSize, user_opt.outputDim, hw_opt.outputDim, stream);
        g = dloss_.as<half>();
    }
    run_backward(g, batchSize, stream);
}

void TinyMLPHashGrid::reset_step() { current_step = 0; }

void TinyMLPHashGrid::step(float lr, float beta1, float beta2, float epsilon, float loss_scale, cudaStream_t stream) {
    if (!m_isTraining) throw std::runtime_error("step called while in inference mode!");
    if (current_step < 50000) current_step++;
    float bc1 = 1.0f - std::pow(beta1, (float)current_step);
    float bc2 = 1.0f - std::pow(beta2, (float)current_step);
    float ils = 1.0f / loss_scale;
    if (off_w_ == off_hash_ + n_hash_) {
        // table and network are adjacent: one launch, sparse rule on the table, dense rule behind it
        nb::throw_on_error(nb_adam_step(arena_->W(off_hash_), arena_->Wh(off_hash_), arena_->G(off_hash_), arena_->M(off_hash_), arena_->V(off_hash_),
                                        n_hash_, n_hash_ + n_w_ + n_b_, lr, beta1, beta2, epsilon, bc1, bc2, ils, 0, stream), "TinyMLPHashGrid::step");
    } else {
        nb::throw_on_error(nb_adam_step(arena_->W(off_hash_), arena_->Wh(off_hash_), arena_->G(off_hash_), arena_->M(off_hash_), arena_->V(off_hash_),
                                        n_hash_, n_hash_, lr, beta1, beta2, epsilon, bc1, bc2, ils, 0, stream), "TinyMLPHashGrid::step (table)");
        nb::throw_on_error(nb_adam_step(arena_->W(off_w_), arena_->Wh(off_w_), arena_->G(off_w_), arena_->M(off_w_), arena_->V(off_w_), 0, n_w_ + n_b_,
                                        lr, beta1, beta2, epsilon, bc1, bc2, ils, 0, stream), "TinyMLPHashGrid::step (network)");
    }
}

void TinyMLPHashGrid::loadWeights(const std::string& filename) {
    std::ifstream in(filename, std::ios::binary);
    if (!in.is_open()) throw std::runtime_error("Cannot open: " + filename);
    MLPGridOptions fopt;
    in.read(reinterpret_cast<char*>(&fopt), sizeof(MLPGridOptions));
    if (fopt.numLevels != hw_opt.numLevels || fopt.tableSize != hw_opt.tableSize || fopt.featuresLevel != hw_opt.featuresLevel ||
        fopt.hiddenDim != hw_opt.hiddenDim || fopt.outputDim != hw_opt.outputDim || fopt.numLayers != hw_opt.numLayers)
        throw std::runtime_error("Weight file dimension mismatch");
    std::vector<float> h((size_t)n_hash_), w((size_t)n_w_), b((size_t)n_b_);
    in.read(reinterpret_cast<char*>(h.data()), (std::streamsize)(n_hash_ * sizeof(float)));
    size_t wo = 0, bo = 0;
    for (int l = 0; l < mlp_opt.numLayers; l++) {
        size_t we = (size_t)g_in(mlp_opt, l) * g_out(mlp_opt, l), be = (size_t)g_out(mlp_opt, l);
        in.read(reinterpret_cast<char*>(w.data() + wo), we * sizeof(float));
        in.read(reinterpret_cast<char*>(b.data() + bo), be * sizeof(float));
        wo += we; bo += be;
    }
    if (!in) throw std::runtime_error("Weight file truncated: " + filename);
    loadHashgrid(h.data());
    loadWeights(w.data(), b.data());
}

void TinyMLPHashGrid::saveWeights(const std::string& filename) {
    std::ofstream out(filename, std::ios::binary);
    if (!out.is_open()) throw std::runtime_error("Cannot open: " + filename);
    out.write(reinterpret_cast<const char*>(&hw_opt), sizeof(MLPGridOptions));
    std::vector<float> h((size_t)n_hash_), w((size_t)n_w_), b((size_t)n_b_);
    saveHashgrid(h.data());
    saveWeights(w.data(), b.data());
    out.write(reinterpret_cast<const char*>(h.data()), (std::streamsize)(n_hash_ * sizeof(float)));
    size_t wo = 0, bo = 0;
    for (int l = 0; l < mlp_opt.numLayers; l++) {
        size_t we = (size_t)g_in(mlp_opt, l) * g_out(mlp_opt, l), be = (size_t)g_out(mlp_opt, l);
        out.write(reinterpret_cast<const char*>(w.data() + wo), we * sizeof(float));
        out.write(reinterpret_cast<const char*>(b.data() + bo), be * sizeof(float));
        wo += we; bo += be;
    }
}

void TinyMLPHashGrid::loadWeights(const float* hw, const float* hb) {
    arena_->upload(off_w_, hw, n_w_);
    arena_->upload(off_b_, hb, n_b_);
}

void TinyMLPHashGrid::saveWeights(float* hw, float* hb) {
    nb::throw_on_cuda(cudaDeviceSynchronize(), "saveWeights");
    arena_->download(off_w_, hw, n_w_);
    arena_->download(off_b_, hb, n_b_);
}

void TinyMLPHashGrid::loadHashgrid(const float* host_hashgrid) { arena_->upload(off_hash_, host_hashgrid, n_hash_); }

void TinyMLPHashGrid::saveHashgrid(float* host_hashgrid) {
    nb::throw_on_cuda(cudaDeviceSynchronize(), "saveHashgrid");
    arena_->download(off_hash_, host_hashgrid, n_hash_);
}
