#include "adam.h"

#include <cmath>
#include <fstream>
#include <stdexcept>

#include "mft_cuda.h"

namespace ops {

using detail::check;
using detail::stream;

float Optimizer::compute_grad_norm(const std::vector<TensorPtr>& parameters) {
    detail::ensure_runtime();
    // one device accumulator for all tensors, one read-back
    auto acc = std::make_shared<Tensor>(std::vector<int64_t>{1}, kFloat32, kCPU);
    float* sum = (float*)acc->device_write();
    check(mft_memset(sum, 0, 4, stream()), "grad norm");
    for (auto& p : parameters) {
        if (!p || !p->grad()) continue;
        auto g = p->grad();
        check(mft_grad_sqnorm_add((const float*)g->device_read(), g->numel(), sum, stream()), "grad norm");
    }
    return std::sqrt(static_cast<const Tensor&>(*acc).data<float>()[0]);
}
void Optimizer::scale_gradients(const std::vector<TensorPtr>& parameters, float scale) {
    for (auto& p : parameters)
        if (p && p->grad()) check(mft_scale_f32((float*)p->grad()->device_readwrite(), scale, p->grad()->numel(), stream()), "scale gradients");
}
void Optimizer::clip_grad_norm(const std::vector<TensorPtr>& parameters, float max_norm) {
    const float norm = compute_grad_norm(parameters);
    if (norm > max_norm) scale_gradients(parameters, max_norm / norm);
}

void Adam::step(const std::vector<TensorPtr>& parameters, const std::vector<TensorPtr>& gradients) {
    if (parameters.size() != gradients.size()) throw std::runtime_error("Parameters and gradients size mismatch");
    if (adam_config_.amsgrad) throw std::runtime_error("Adam: the AMSGrad variant is not available on this backend");
    for (size_t i = 0; i < parameters.size(); ++i) {
        const auto& p = parameters[i];
        const auto& g = gradients[i];
        if (!g) continue;                                   // parameters without a gradient are skipped, their step counter too
        auto& st = states_[p];
        if (st.m.empty()) {
            st.m.push_back(std::make_shared<Tensor>(p->shape(), kFloat32, kCPU));
            st.v.push_back(std::make_shared<Tensor>(p->shape(), kFloat32, kCPU));
        }
        st.step++;
        check(mft_adam_step((float*)p->device_readwrite(), (float*)g->device_readwrite(), (float*)st.m[0]->device_readwrite(),
                            (float*)st.v[0]->device_readwrite(), p->numel(), (int64_t)st.step, adam_config_.learning_rate, adam_config_.beta1,
                            adam_config_.beta2, adam_config_.epsilon, adam_config_.weight_decay, nullptr, 0.f, 0.f, 0, stream()), "Adam::step");
    }
}

void Adam::save_state(const std::string& path) const {
    std::ofstream f(path, std::ios::binary);
    if (!f.is_open()) throw std::runtime_error("Failed to open file for saving Adam state: " + path);
    const uint64_t n = states_.size();
    f.write(reinterpret_cast<const char*>(&n), sizeof n);
}
void Adam::load_state(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f.is_open()) throw std::runtime_error("Failed to open file for loading Adam state: " + path);
    // like the reference, only the header is read: moments are rebuilt from the next steps
}

}  // namespace ops
