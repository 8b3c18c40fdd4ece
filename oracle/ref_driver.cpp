// Test infrastructure, not product code.
//
// Driver that runs the UNMODIFIED reference CPU implementation of the LoRA
// fine-tuning step (linked from the reference's own sources by oracle/Makefile)
// on inputs read from a case directory, and dumps its results as .npy files.
// It only calls the reference's public C++ API; all arithmetic is the
// reference's.  Used by tests/ to produce golden vectors, as the parity checker
// on the GPU box, and as the timed CPU baseline of bench.py.
//
//   ref_driver shapes <case_dir>   list parameters() / trainable_parameters()
//   ref_driver model  <case_dir>   forward + lm_cross_entropy + backward
//                                  (+ clip + Adam) on a whole model
//   ref_driver op     <case_dir>   one operator (or operator chain) fwd + bwd
//
// Case directory layout: `case.txt` holds `key value` lines; tensors are .npy
// files (little-endian float32 / int32, C order); results go to <case_dir>/out.
#include "finetune_ops/core/tensor.h"
#include "finetune_ops/core/ops.h"
#include "finetune_ops/core/lm_loss.h"
#include "finetune_ops/core/autograd_engine.h"
#include "finetune_ops/core/memory_efficient_attention.h"
#include "finetune_ops/nn/lora_linear.h"
#include "finetune_ops/graph/auto_model.h"
#include "finetune_ops/optim/adam.h"

#include <chrono>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <iostream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <sys/stat.h>

#ifdef USE_BLAS
#include <cblas.h>
#endif

using ops::TensorPtr;
using Shape = std::vector<int64_t>;

// ---------------------------------------------------------------- npy I/O
static TensorPtr npy_load(const std::string& path) {
    std::ifstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot open " + path);
    char magic[6]; f.read(magic, 6);
    if (std::memcmp(magic, "\x93NUMPY", 6) != 0) throw std::runtime_error("not npy: " + path);
    unsigned char ver[2]; f.read((char*)ver, 2);
    uint32_t hlen = 0;
    if (ver[0] == 1) { uint16_t h; f.read((char*)&h, 2); hlen = h; }
    else { f.read((char*)&hlen, 4); }
    std::string hdr(hlen, ' '); f.read(&hdr[0], hlen);
    auto dpos = hdr.find("'descr'");
    auto q1 = hdr.find('\'', dpos + 7); auto q2 = hdr.find('\'', q1 + 1);
    std::string descr = hdr.substr(q1 + 1, q2 - q1 - 1);
    if (hdr.find("'fortran_order': True") != std::string::npos) throw std::runtime_error("fortran npy");
    auto spos = hdr.find("'shape'");
    auto p1 = hdr.find('(', spos); auto p2 = hdr.find(')', p1);
    std::string sh = hdr.substr(p1 + 1, p2 - p1 - 1);
    Shape shape; std::stringstream ss(sh); std::string tok;
    while (std::getline(ss, tok, ',')) {
        bool digit = false; for (char c : tok) if (isdigit((unsigned char)c)) digit = true;
        if (digit) shape.push_back(std::stoll(tok));
    }
    if (shape.empty()) shape.push_back(1);
    ops::DType dt;
    if (descr == "<f4") dt = ops::kFloat32;
    else if (descr == "<i4") dt = ops::kInt32;
    else throw std::runtime_error("unsupported npy dtype " + descr + " in " + path);
    auto t = std::make_shared<ops::Tensor>(shape, dt, ops::kCPU);
    f.read((char*)t->data_ptr(), (std::streamsize)(t->numel() * 4));
    if (!f) throw std::runtime_error("short read " + path);
    return t;
}

static void npy_save_raw(const std::string& path, const void* data, const Shape& shape, const char* descr) {
    std::string hdr = std::string("{'descr': '") + descr + "', 'fortran_order': False, 'shape': (";
    for (size_t i = 0; i < shape.size(); ++i) { hdr += std::to_string(shape[i]); hdr += (shape.size() == 1 || i + 1 < shape.size()) ? "," : ""; }
    hdr += "), }";
    while ((10 + hdr.size() + 1) % 64 != 0) hdr += ' ';
    hdr += '\n';
    std::ofstream f(path, std::ios::binary);
    if (!f) throw std::runtime_error("cannot write " + path);
    f.write("\x93NUMPY\x01\x00", 8);
    uint16_t h = (uint16_t)hdr.size(); f.write((char*)&h, 2);
    f.write(hdr.data(), (std::streamsize)hdr.size());
    int64_t n = 1; for (auto d : shape) n *= d;
    f.write((const char*)data, (std::streamsize)(n * 4));
}
static void npy_save(const std::string& path, const TensorPtr& t) {
    if (!t) return;
    npy_save_raw(path, t->data_ptr(), t->shape(), t->dtype() == ops::kInt32 ? "<i4" : "<f4");
}
static bool file_exists(const std::string& p) { struct stat st; return stat(p.c_str(), &st) == 0; }

// ---------------------------------------------------------------- case.txt
struct Case {
    std::string dir;
    std::map<std::string, std::string> kv;
    bool has(const std::string& k) const { return kv.count(k) > 0; }
    std::string s(const std::string& k, const std::string& d = "") const { auto it = kv.find(k); return it == kv.end() ? d : it->second; }
    double f(const std::string& k, double d) const { auto it = kv.find(k); return it == kv.end() ? d : std::stod(it->second); }
    long i(const std::string& k, long d) const { auto it = kv.find(k); return it == kv.end() ? d : std::stol(it->second); }
    TensorPtr in(const std::string& name) const { return npy_load(dir + "/" + name + ".npy"); }
    bool has_in(const std::string& name) const { return file_exists(dir + "/" + name + ".npy"); }
    void out(const std::string& name, const TensorPtr& t) const { npy_save(dir + "/out/" + name + ".npy", t); }
};
static Case load_case(const std::string& dir) {
    Case c; c.dir = dir;
    std::ifstream f(dir + "/case.txt");
    if (!f) throw std::runtime_error("missing case.txt in " + dir);
    std::string line;
    while (std::getline(f, line)) {
        if (line.empty() || line[0] == '#') continue;
        auto sp = line.find(' ');
        if (sp == std::string::npos) { c.kv[line] = ""; continue; }
        c.kv[line.substr(0, sp)] = line.substr(sp + 1);
    }
    mkdir((dir + "/out").c_str(), 0755);
    return c;
}
static double now_s() {
    return std::chrono::duration<double>(std::chrono::steady_clock::now().time_since_epoch()).count();
}
static TensorPtr grad_leaf(const TensorPtr& t) { t->set_requires_grad(true); return t; }
static std::string idx3(size_t i) { char b[16]; snprintf(b, sizeof b, "%04zu", i); return b; }

// ---------------------------------------------------------------- model mode
static std::vector<std::string> split_csv(const std::string& s) {
    std::vector<std::string> out; std::stringstream ss(s); std::string t;
    while (std::getline(ss, t, ',')) if (!t.empty()) out.push_back(t);
    return out;
}

struct ModelHolder {
    std::unique_ptr<ops::AutoModelForCausalLM> model;
    std::unique_ptr<ops::LoraInjector> gpt2_injector;   // used when GPT-2 LoRA is injected with split_qkv=0
    std::vector<TensorPtr> trainables() {
        return model->trainable_parameters();
    }
};

static void init_lora(ModelHolder& mh, const Case& c) {
    ops::AutoLoraConfig lc;
    lc.rank = (int)c.i("lora_rank", 8);
    lc.alpha = (float)c.f("lora_alpha", 16.0);
    lc.dropout = 0.0f;
    lc.seed = 42;
    lc.target_modules = split_csv(c.s("lora_targets", ""));
    if (mh.model->family() == ops::ModelFamily::GPT2 && c.i("gpt2_split_qkv", 0) == 0) {
        // The example CLI injects with split_qkv=false; AutoModel would use true.
        ops::LoraSpec spec;
        spec.rank = lc.rank; spec.alpha = lc.alpha; spec.dropout = 0.0f; spec.split_qkv = false;
        spec.targets.clear();
        for (auto& m : lc.target_modules) {
            if (m == "c_attn") spec.targets.push_back(ops::LoraTarget::AttnQKV);
            else if (m == "c_proj") spec.targets.push_back(ops::LoraTarget::AttnProj);
            else if (m == "c_fc") spec.targets.push_back(ops::LoraTarget::MlpFcIn);
            else if (m == "mlp_c_proj") spec.targets.push_back(ops::LoraTarget::MlpFcOut);
        }
        if (spec.targets.empty()) spec.targets = {ops::LoraTarget::AttnQKV, ops::LoraTarget::AttnProj};
        mh.model->gpt2()->init_lora_modules();
        mh.gpt2_injector = std::make_unique<ops::LoraInjector>();
        mh.gpt2_injector->inject(*mh.model->gpt2(), spec);
    } else {
        mh.model->init_lora(lc);
    }
}

static ModelHolder build_model(const Case& c, bool load_values) {
    ModelHolder mh;
    ops::AutoModelLoadOptions opt; opt.load_weights = false; opt.verbose = false;
    mh.model = ops::AutoModelForCausalLM::from_pretrained(c.dir, opt);
    auto params = mh.model->parameters();
    if (load_values) {
        for (size_t i = 0; i < params.size(); ++i) {
            auto src = npy_load(c.dir + "/params/" + idx3(i) + ".npy");
            if (src->numel() != params[i]->numel())
                throw std::runtime_error("param " + std::to_string(i) + " size mismatch");
            std::memcpy(params[i]->data_ptr(), src->data_ptr(), (size_t)src->numel() * 4);
        }
    }
    init_lora(mh, c);
    auto tr = mh.trainables();
    if (load_values) {
        for (size_t i = 0; i < tr.size(); ++i) {
            auto src = npy_load(c.dir + "/lora/" + idx3(i) + ".npy");
            if (src->numel() != tr[i]->numel())
                throw std::runtime_error("lora " + std::to_string(i) + " size mismatch");
            std::memcpy(tr[i]->data_ptr(), src->data_ptr(), (size_t)src->numel() * 4);
        }
    }
    return mh;
}

static int run_shapes(const Case& c) {
    auto mh = build_model(c, false);
    std::ofstream f(c.dir + "/out/shapes.txt");
    auto dump = [&](const char* tag, const std::vector<TensorPtr>& v) {
        for (size_t i = 0; i < v.size(); ++i) {
            f << tag << " " << i;
            if (v[i]) for (auto d : v[i]->shape()) f << " " << d;
            f << "\n";
        }
    };
    dump("param", mh.model->parameters());
    dump("lora", mh.trainables());
    return 0;
}

static int run_model(const Case& c) {
    auto mh = build_model(c, true);
    auto ids = c.in("input_ids");
    auto labels = c.in("labels");
    TensorPtr mask = c.has_in("attention_mask") ? c.in("attention_mask") : nullptr;
    const int steps = (int)c.i("steps", 1);
    const float max_norm = (float)c.f("max_grad_norm", 0.0);   // 0 = no clipping
    ops::AdamConfig ac((float)c.f("lr", 2e-4), (float)c.f("beta1", 0.9), (float)c.f("beta2", 0.999),
                       (float)c.f("eps", 1e-8), (float)c.f("weight_decay", 0.0));
    ops::Adam adam(ac);
    const bool dump_logits = c.i("dump_logits", 0) != 0;
    const bool do_update = c.i("update", 1) != 0;
    std::ofstream tf(c.dir + "/out/timing.txt");
    std::vector<float> losses;
    for (int step = 0; step < steps; ++step) {
        auto params = mh.trainables();
        double t0 = now_s();
        auto logits = mh.model->forward(ids, mask);
        double t1 = now_s();
        auto loss = ops::lm_cross_entropy(logits, labels, -100, "mean");
        double t2 = now_s();
        loss->backward();
        double t3 = now_s();
        losses.push_back(loss->data<float>()[0]);
        if (step == 0) {
            if (dump_logits) c.out("logits", logits);
            for (size_t i = 0; i < params.size(); ++i)
                if (params[i]->grad()) c.out("grad_" + idx3(i), params[i]->grad());
        }
        logits.reset();
        double t4 = now_s();
        if (do_update) {
            if (max_norm > 0.0f) adam.clip_grad_norm(params, max_norm);
            std::vector<TensorPtr> grads;
            for (auto& p : params) grads.push_back(p->grad());
            adam.step(params, grads);
            adam.zero_grad(params);
        }
        double t5 = now_s();
        tf << "step " << step << " forward " << (t1 - t0) << " loss " << (t2 - t1) << " backward " << (t3 - t2)
           << " update " << (t5 - t4) << " total " << (t3 - t0) + (t5 - t4) << "\n";
        tf.flush();
    }
    auto params = mh.trainables();
    for (size_t i = 0; i < params.size(); ++i) c.out("lora_after_" + idx3(i), params[i]);
    npy_save_raw(c.dir + "/out/loss.npy", losses.data(), {(int64_t)losses.size()}, "<f4");
    return 0;
}

// ---------------------------------------------------------------- op mode
static TensorPtr build_mask(int64_t S, int64_t window) {
    // Additive mask as the reference graphs build it: 0 where key j is visible to
    // query i, -1e10 elsewhere (causal: j<=i; sliding: additionally i-j < window).
    auto m = ops::zeros({1, 1, S, S});
    float* d = m->data<float>();
    for (int64_t i = 0; i < S; ++i)
        for (int64_t j = 0; j < S; ++j) {
            bool ok = j <= i && (window <= 0 || i - j < window);
            d[i * S + j] = ok ? 0.0f : -1e10f;
        }
    return m;
}

static int run_op(const Case& c) {
    const std::string op = c.s("op");
    double t0 = now_s(), t1 = t0, t2 = t0;
    if (op == "attention") {
        // repeat_kv -> transpose -> matmul -> mul(scale) -> add(mask) -> softmax -> matmul
        auto q = grad_leaf(c.in("q")), k = grad_leaf(c.in("k")), v = grad_leaf(c.in("v"));
        auto dO = c.in("dO");
        int64_t nh = q->shape()[1], nkv = k->shape()[1], S = q->shape()[2], hd = q->shape()[3];
        float scale = (float)c.f("scale", 1.0 / std::sqrt((double)hd));
        float theta = (float)c.f("rope_theta", 0.0);
        auto mask = build_mask(S, c.i("window", 0));
        t0 = now_s();
        TensorPtr qu = q, ku = k;
        if (theta > 0) { qu = ops::apply_rope(q, (int)S, (int)hd, theta); ku = ops::apply_rope(k, (int)S, (int)hd, theta); }
        auto kf = ops::repeat_kv_heads(ku, (int)(nh / nkv));
        auto vf = ops::repeat_kv_heads(v, (int)(nh / nkv));
        auto scores = ops::mul(ops::matmul(qu, ops::transpose(kf, 2, 3)), scale);
        scores = ops::add(scores, mask);
        auto probs = ops::softmax(scores, -1);
        auto out = ops::matmul(probs, vf);
        t1 = now_s();
        ops::autograd::Engine::instance().run_backward({out}, {dO});
        t2 = now_s();
        c.out("O", out); c.out("dQ", q->grad()); c.out("dK", k->grad()); c.out("dV", v->grad());
    } else if (op == "lora_linear") {
        auto x = grad_leaf(c.in("x"));
        auto W = c.in("W");
        TensorPtr bias = c.has_in("bias") ? c.in("bias") : nullptr;
        auto A = grad_leaf(c.in("A")), B = grad_leaf(c.in("B"));
        auto dY = c.in("dY");
        ops::LoRALinear lin(W, bias);
        lin.attach_lora(A, B, (float)c.f("scale", 2.0));
        t0 = now_s();
        auto y = lin.forward(x);
        t1 = now_s();
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        t2 = now_s();
        c.out("y", y); c.out("dx", x->grad()); c.out("dA", A->grad()); c.out("dB", B->grad());
    } else if (op == "matmul" || op == "matmul_rhs_T") {
        auto a = grad_leaf(c.in("a")); auto b = c.in("b");
        auto dY = c.in("dY");
        t0 = now_s();
        auto y = op == "matmul" ? ops::matmul(a, b) : ops::matmul_rhs_T(a, b);
        t1 = now_s();
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        t2 = now_s();
        c.out("y", y); c.out("da", a->grad());
    } else if (op == "rms_norm" || op == "rms_norm_affine") {
        auto x = grad_leaf(c.in("x")), w = grad_leaf(c.in("w"));
        auto dY = c.in("dY");
        float eps = (float)c.f("eps", 1e-6);
        t0 = now_s();
        auto y = op == "rms_norm" ? ops::rms_norm(x, w, eps) : ops::rms_norm_affine(x, w, eps);
        t1 = now_s();
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        t2 = now_s();
        c.out("y", y); c.out("dx", x->grad()); c.out("dw", w->grad());
    } else if (op == "layer_norm") {
        auto x = grad_leaf(c.in("x")), w = grad_leaf(c.in("w")), b = grad_leaf(c.in("b"));
        auto dY = c.in("dY");
        t0 = now_s();
        auto y = ops::layer_norm(x, w, b, (float)c.f("eps", 1e-5));
        t1 = now_s();
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        t2 = now_s();
        c.out("y", y); c.out("dx", x->grad()); c.out("dw", w->grad()); c.out("db", b->grad());
    } else if (op == "gelu") {
        auto x = grad_leaf(c.in("x")); auto dY = c.in("dY");
        auto y = ops::gelu(x);
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        c.out("y", y); c.out("dx", x->grad());
    } else if (op == "swiglu" || op == "geglu") {
        auto g = grad_leaf(c.in("gate")), u = grad_leaf(c.in("up")); auto dY = c.in("dY");
        auto y = op == "swiglu" ? ops::swiglu(g, u) : ops::mul(ops::gelu(g), u);
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        c.out("y", y); c.out("dgate", g->grad()); c.out("dup", u->grad());
    } else if (op == "rope") {
        auto x = grad_leaf(c.in("x")); auto dY = c.in("dY");
        int64_t S = x->shape()[2], hd = x->shape()[3];
        auto y = ops::apply_rope(x, (int)S, (int)hd, (float)c.f("rope_theta", 10000.0));
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        c.out("y", y); c.out("dx", x->grad());
    } else if (op == "repeat_kv") {
        auto x = grad_leaf(c.in("x")); auto dY = c.in("dY");
        auto y = ops::repeat_kv_heads(x, (int)c.i("repeat", 1));
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        c.out("y", y); c.out("dx", x->grad());
    } else if (op == "add") {
        auto a = grad_leaf(c.in("a")), b = grad_leaf(c.in("b")); auto dY = c.in("dY");
        auto y = ops::add(a, b);
        ops::autograd::Engine::instance().run_backward({y}, {dY});
        c.out("y", y); c.out("da", a->grad()); c.out("db", b->grad());
    } else if (op == "lm_ce") {
        // dense logits path: loss + d(logits)
        auto logits = grad_leaf(c.in("logits")); auto labels = c.in("labels");
        t0 = now_s();
        auto loss = ops::lm_cross_entropy(logits, labels, (int)c.i("ignore_index", -100), c.s("reduction", "mean"));
        t1 = now_s();
        loss->backward();
        t2 = now_s();
        c.out("loss", loss); c.out("dlogits", logits->grad());
    } else if (op == "lm_head_ce") {
        // hidden [B,S,H] x tied table W [V,H] -> logits -> loss ; d(hidden)
        auto hid = grad_leaf(c.in("hidden")); auto W = c.in("W"); auto labels = c.in("labels");
        t0 = now_s();
        auto logits = ops::matmul_rhs_T(hid, W);
        auto loss = ops::lm_cross_entropy(logits, labels, (int)c.i("ignore_index", -100), c.s("reduction", "mean"));
        t1 = now_s();
        loss->backward();
        t2 = now_s();
        c.out("loss", loss); c.out("dhidden", hid->grad());
    } else if (op == "streaming_ce") {
        auto hid = grad_leaf(c.in("hidden")); auto W = c.in("W"); auto labels = c.in("labels");
        t0 = now_s();
        auto loss = ops::streaming_lm_cross_entropy(hid, W, labels, (int)c.i("ignore_index", -100), c.s("reduction", "mean"));
        t1 = now_s();
        loss->backward();
        t2 = now_s();
        c.out("loss", loss); c.out("dhidden", hid->grad());
    } else if (op == "adam") {
        // `steps` Adam updates of one parameter tensor with given per-step gradients g0,g1,...
        auto p = grad_leaf(c.in("p"));
        ops::AdamConfig ac((float)c.f("lr", 1e-3), (float)c.f("beta1", 0.9), (float)c.f("beta2", 0.999),
                           (float)c.f("eps", 1e-8), (float)c.f("weight_decay", 0.0));
        ops::Adam adam(ac);
        float max_norm = (float)c.f("max_grad_norm", 0.0);
        int steps = (int)c.i("steps", 1);
        for (int s = 0; s < steps; ++s) {
            auto g = c.in("g" + std::to_string(s));
            p->set_grad(g);
            if (max_norm > 0) adam.clip_grad_norm({p}, max_norm);
            adam.step({p}, {p->grad()});
        }
        c.out("p", p);
    } else {
        throw std::runtime_error("unknown op " + op);
    }
    std::ofstream tf(c.dir + "/out/timing.txt");
    tf << "forward " << (t1 - t0) << " backward " << (t2 - t1) << "\n";
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 3) { std::fprintf(stderr, "usage: ref_driver shapes|model|op <case_dir>\n"); return 2; }
    try {
#ifdef USE_BLAS
        if (const char* nt = std::getenv("ORACLE_BLAS_THREADS")) openblas_set_num_threads(std::atoi(nt));
#endif
        std::string mode = argv[1];
        Case c = load_case(argv[2]);
        if (mode == "shapes") return run_shapes(c);
        if (mode == "model") return run_model(c);
        if (mode == "op") return run_op(c);
        std::fprintf(stderr, "unknown mode %s\n", mode.c_str());
        return 2;
    } catch (const std::exception& e) {
        std::fprintf(stderr, "ref_driver error: %s\n", e.what());
        return 1;
    }
}
