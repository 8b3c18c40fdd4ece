#include "lora_saver.h"

#include <algorithm>
#include <cctype>
#include <iostream>
#include <map>
#include <set>
#include <sstream>
#include <stdexcept>

#include "mft_step.h"
#include "lora_file.h"

namespace ops {

namespace detail {

void write_adapter_file(const std::string& path, const std::map<std::string, TensorPtr>& tensors, const std::map<std::string, std::string>& metadata) {
    std::vector<const char*> names, mk, mv;
    std::vector<int32_t> ndims;
    std::vector<int64_t> shapes;
    std::vector<const float*> data;
    for (const auto& kv : tensors) {
        const Tensor& t = *kv.second;
        if (t.dtype() != kFloat32 || t.shape().size() > 8) throw std::runtime_error("adapter file: tensors must be float32 with at most 8 dimensions");
        names.push_back(kv.first.c_str());
        ndims.push_back((int32_t)t.shape().size());
        for (int d = 0; d < 8; ++d) shapes.push_back(d < (int)t.shape().size() ? t.shape()[(size_t)d] : 1);
        data.push_back(t.data<float>());                       // const access: brings the host copy up to date
    }
    for (const auto& kv : metadata) { mk.push_back(kv.first.c_str()); mv.push_back(kv.second.c_str()); }
    if (mft_safetensors_write_f32(path.c_str(), (int32_t)names.size(), names.data(), ndims.data(), shapes.data(), data.data(), (int32_t)mk.size(),
                                  mk.data(), mv.data()) != MFT_OK)
        throw std::runtime_error("cannot write " + path + ": " + mft_last_error());
}

std::map<std::string, TensorPtr> read_adapter_file(const std::string& path, std::map<std::string, std::string>* metadata) {
    mft_safetensors_t* h = nullptr;
    if (mft_safetensors_open(path.c_str(), &h) != MFT_OK) throw std::runtime_error("cannot open " + path + ": " + mft_last_error());
    std::map<std::string, TensorPtr> out;
    try {
        if (metadata)
            for (auto& kv : *metadata)
                if (const char* v = mft_safetensors_metadata(h, kv.first.c_str())) kv.second = v;
        const int64_t n = mft_safetensors_count(h);
        for (int64_t i = 0; i < n; ++i) {
            const std::string name = mft_safetensors_name(h, i);
            char dtype[8] = {0};
            int32_t nd = 0;
            int64_t shape[8] = {0};
            if (mft_safetensors_info(h, name.c_str(), dtype, &nd, shape) != MFT_OK) throw std::runtime_error(mft_last_error());
            auto t = std::make_shared<Tensor>(std::vector<int64_t>(shape, shape + nd), kFloat32, kCPU);
            if (mft_safetensors_read_f32(h, name.c_str(), t->data<float>(), 0) != MFT_OK) throw std::runtime_error(mft_last_error());
            out[name] = t;
        }
    } catch (...) {
        mft_safetensors_close(h);
        throw;
    }
    mft_safetensors_close(h);
    return out;
}

}  // namespace detail

namespace {
const char* target_name(LoraTarget t) {
    switch (t) {
        case LoraTarget::AttnQKV: return "AttnQKV";
        case LoraTarget::AttnProj: return "AttnProj";
        case LoraTarget::MlpFcIn: return "MlpFcIn";
        default: return "MlpFcOut";
    }
}
bool name_target(std::string s, LoraTarget* out) {
    s.erase(std::remove(s.begin(), s.end(), '_'), s.end());
    std::transform(s.begin(), s.end(), s.begin(), [](unsigned char c) { return (char)std::tolower(c); });
    if (s == "attnqkv") *out = LoraTarget::AttnQKV;
    else if (s == "attnproj") *out = LoraTarget::AttnProj;
    else if (s == "mlpfcin") *out = LoraTarget::MlpFcIn;
    else if (s == "mlpfcout") *out = LoraTarget::MlpFcOut;
    else return false;
    return true;
}
bool key_target(const std::string& k, LoraTarget* out) {
    if (k == "attn.q" || k == "attn.k" || k == "attn.v" || k == "attn.qkv") *out = LoraTarget::AttnQKV;
    else if (k == "attn.proj") *out = LoraTarget::AttnProj;
    else if (k == "mlp.fc_in") *out = LoraTarget::MlpFcIn;
    else if (k == "mlp.fc_out") *out = LoraTarget::MlpFcOut;
    else return false;
    return true;
}
std::string num(float v) { std::ostringstream os; os << v; return os.str(); }
}  // namespace

bool LoRAState::compatible_with(const GPT2Model&) const {
    if (rank < 1 || rank > 128) return false;
    return !tensors.empty();
}

std::string LoraSaver::make_peft_key(int layer, const std::string& target, const std::string& ab) {
    return "layer." + std::to_string(layer) + "." + target + ".lora_" + ab;
}

bool LoraSaver::parse_peft_key(const std::string& key, int& layer, std::string& target, std::string& ab) {
    const size_t lp = key.find("layer."), ap = key.find(".lora_");
    if (lp == std::string::npos || ap == std::string::npos) return false;
    const size_t s = lp + 6, e = key.find('.', s);
    if (e == std::string::npos || e >= ap) return false;
    try { layer = std::stoi(key.substr(s, e - s)); } catch (...) { return false; }
    target = key.substr(e + 1, ap - e - 1);
    const std::string tail = key.substr(ap + 6);
    if (tail != "A" && tail != "B") return false;
    ab = tail;
    return true;
}

void LoraSaver::save_safetensors(const std::string& path, const GPT2Model& model, const LoraSpec& spec) {
    std::map<std::string, TensorPtr> state;
    auto wanted = [&](LoraTarget t) { return spec.targets.empty() || std::find(spec.targets.begin(), spec.targets.end(), t) != spec.targets.end(); };
    for (int i = 0; i < model.config().n_layer; ++i) {
        const GPT2BlockWeights& b = model.get_block(i);
        auto put = [&](const std::string& name, const LoRASlice& s) {
            if (!s.A || !s.B) return;
            state[make_peft_key(i, name, "A")] = s.A;
            state[make_peft_key(i, name, "B")] = s.B;
        };
        if (b.qkv_lin && wanted(LoraTarget::AttnQKV) && !b.qkv_lin->slices().empty()) {
            const auto& sl = b.qkv_lin->slices();
            if (spec.split_qkv) {
                static const char* parts[] = {"attn.q", "attn.k", "attn.v"};
                for (size_t k = 0; k < std::min<size_t>(sl.size(), 3); ++k) put(parts[k], sl[k]);
            } else {
                put("attn.qkv", sl.front());
            }
        }
        if (b.proj_lin && wanted(LoraTarget::AttnProj) && !b.proj_lin->slices().empty()) put("attn.proj", b.proj_lin->slices().front());
        if (b.fc_in_lin && wanted(LoraTarget::MlpFcIn) && !b.fc_in_lin->slices().empty()) put("mlp.fc_in", b.fc_in_lin->slices().front());
        if (b.fc_out_lin && wanted(LoraTarget::MlpFcOut) && !b.fc_out_lin->slices().empty()) put("mlp.fc_out", b.fc_out_lin->slices().front());
    }
    std::string targets;
    for (size_t i = 0; i < spec.targets.size(); ++i) targets += (i ? "," : "") + std::string(target_name(spec.targets[i]));
    detail::write_adapter_file(path, state, {{"rank", std::to_string(spec.rank)}, {"alpha", num(spec.alpha)}, {"dropout", num(spec.dropout)},
                                             {"split_qkv", spec.split_qkv ? "true" : "false"}, {"targets", targets}});
    std::cout << "[LoraSaver] Saved " << state.size() << " tensors to " << path << std::endl;
}

LoRAState LoraSaver::load_safetensors(const std::string& path) {
    std::map<std::string, std::string> meta = {{"rank", ""}, {"alpha", ""}, {"dropout", ""}, {"split_qkv", ""}, {"targets", ""}};
    auto tensors = detail::read_adapter_file(path, &meta);
    LoRAState st;
    st.rank = 0;
    try { if (!meta["rank"].empty()) st.rank = std::stoi(meta["rank"]); } catch (...) {}
    try { if (!meta["alpha"].empty()) st.alpha = std::stof(meta["alpha"]); } catch (...) {}
    try { if (!meta["dropout"].empty()) st.dropout = std::stof(meta["dropout"]); } catch (...) {}
    if (!meta["split_qkv"].empty()) st.split_qkv = meta["split_qkv"] == "true" || meta["split_qkv"] == "1" || meta["split_qkv"] == "True";
    std::stringstream ss(meta["targets"]);
    for (std::string item; std::getline(ss, item, ',');) {
        LoraTarget t;
        if (name_target(item, &t) && std::find(st.targets.begin(), st.targets.end(), t) == st.targets.end()) st.targets.push_back(t);
    }
    bool fused = false, split = false;
    std::set<LoraTarget> seen;
    for (auto& kv : tensors) {
        st.tensors[kv.first] = kv.second;
        int layer; std::string target, ab;
        if (!parse_peft_key(kv.first, layer, target, ab)) continue;
        if (st.rank <= 0 && ab == "A" && kv.second->shape().size() == 2) st.rank = (int)kv.second->shape()[1];     // A is [in, rank]
        fused = fused || target == "attn.qkv";
        split = split || target == "attn.q" || target == "attn.k" || target == "attn.v";
        LoraTarget t;
        if (key_target(target, &t)) seen.insert(t);
    }
    if (st.rank <= 0) st.rank = 8;
    if (st.targets.empty()) st.targets.assign(seen.begin(), seen.end());
    if (fused) st.split_qkv = false;
    else if (split) st.split_qkv = true;
    std::cout << "[LoraSaver] Loaded " << st.tensors.size() << " LoRA tensors from " << path << " (rank " << st.rank << ", alpha " << st.alpha << ")" << std::endl;
    return st;
}

void LoraSaver::attach_from_state(GPT2Model& model, const LoRAState& state) {
    std::map<std::string, TensorPtr> a, b;
    for (const auto& kv : state.tensors) {
        int layer; std::string target, ab;
        if (!parse_peft_key(kv.first, layer, target, ab)) continue;
        (ab == "A" ? a : b)[std::to_string(layer) + "." + target] = kv.second;
    }
    model.init_lora_modules();
    const int C = model.config().n_embd;
    const float scale = state.alpha / (float)std::max(1, state.rank);
    for (int i = 0; i < model.config().n_layer; ++i) {
        GPT2BlockWeights& blk = model.get_block(i);
        for (LoRALinear* m : {blk.qkv_lin.get(), blk.proj_lin.get(), blk.fc_in_lin.get(), blk.fc_out_lin.get()})
            if (m) m->clear_lora();
        auto attach = [&](const std::string& target, LoRALinear* lin, int col0, int cols) {
            const std::string key = std::to_string(i) + "." + target;
            auto ia = a.find(key), ib = b.find(key);
            if (!lin || ia == a.end() || ib == b.end()) return;
            ia->second->set_requires_grad(true);
            ib->second->set_requires_grad(true);
            lin->attach_lora(ia->second, ib->second, scale, col0, cols);
        };
        attach("attn.qkv", blk.qkv_lin.get(), 0, 3 * C);
        attach("attn.q", blk.qkv_lin.get(), 0, C);
        attach("attn.k", blk.qkv_lin.get(), C, C);
        attach("attn.v", blk.qkv_lin.get(), 2 * C, C);
        attach("attn.proj", blk.proj_lin.get(), 0, C);
        attach("mlp.fc_in", blk.fc_in_lin.get(), 0, 4 * C);
        attach("mlp.fc_out", blk.fc_out_lin.get(), 0, C);
    }
}

}  // namespace ops
