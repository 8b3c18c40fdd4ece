#include "autograd_engine.h"

#include <algorithm>
#include <unordered_map>
#include <unordered_set>

#include "ops.h"

namespace ops {
namespace autograd {

Engine& Engine::instance() {
    static Engine e;
    return e;
}

NodePtr Engine::register_node(const TensorPtr& output, const std::vector<TensorPtr>& inputs, BackwardFunctionPtr fn) {
    if (!enabled_ || !output) return nullptr;
    auto n = std::make_shared<Node>();
    n->owner = output.get();
    n->inputs = inputs;
    n->backward_fn = std::move(fn);
    output->grad_node_ = n;
    output->requires_grad_ = true;
    live_.push_back(n);
    return n;
}

NodePtr Engine::get_node(const TensorPtr& t) { return t ? t->grad_node_ : nullptr; }

void Engine::clear_graph() {
    for (auto& w : live_)
        if (auto n = w.lock()) {
            if (n->owner && n->owner->grad_node_ == n) n->owner->grad_node_ = nullptr;
            n->inputs.clear();
            n->backward_fn.reset();
        }
    live_.clear();
}

static TensorPtr accumulate(const TensorPtr& have, const TensorPtr& g) {
    if (!have) return g;
    return ops::add(have, g);        // out of place: `g` may be shared with another consumer
}

void Engine::run_backward(const std::vector<TensorPtr>& outputs, const std::vector<TensorPtr>& output_grads) {
    NoGradGuard guard;               // backward rules call ops:: but must not record
    // reverse post-order over the nodes reachable from the roots
    std::vector<Node*> order;
    std::unordered_set<Node*> seen;
    std::vector<std::pair<Node*, size_t>> stack;
    for (auto& o : outputs) {
        if (!o || !o->grad_node_ || seen.count(o->grad_node_.get())) continue;
        stack.push_back({o->grad_node_.get(), 0});
        seen.insert(o->grad_node_.get());
        while (!stack.empty()) {
            auto& [n, idx] = stack.back();
            if (idx < n->inputs.size()) {
                const TensorPtr& in = n->inputs[idx++];
                if (in && in->grad_node_ && !seen.count(in->grad_node_.get())) {
                    seen.insert(in->grad_node_.get());
                    stack.push_back({in->grad_node_.get(), 0});
                }
            } else {
                order.push_back(n);
                stack.pop_back();
            }
        }
    }
    std::unordered_map<Node*, TensorPtr> pending;
    auto deliver = [&](const TensorPtr& t, const TensorPtr& g) {
        if (!t || !g || !t->requires_grad_) return;
        if (t->grad_node_) pending[t->grad_node_.get()] = accumulate(pending[t->grad_node_.get()], g);
        else t->grad_ = accumulate(t->grad_, g);               // leaf: accumulates across backward() calls
    };
    for (size_t i = 0; i < outputs.size(); ++i) {
        const TensorPtr& o = outputs[i];
        if (!o) continue;
        TensorPtr g = (i < output_grads.size()) ? output_grads[i] : nullptr;
        if (!g) {
            if (o->numel() != 1) throw TensorError("grad can be implicitly created only for scalar outputs");
            g = ops::ones(o->shape(), o->dtype(), o->device());
        }
        if (g->shape() != o->shape()) throw TensorError("gradient shape does not match tensor shape");
        deliver(o, g);
    }
    for (auto it = order.rbegin(); it != order.rend(); ++it) {
        Node* n = *it;
        auto pg = pending.find(n);
        if (pg == pending.end() || !pg->second) continue;
        TensorPtr g = pg->second;
        if (n->owner && n->owner->retain_grad_) n->owner->grad_ = accumulate(n->owner->grad_, g);
        if (n->backward_fn) {
            std::vector<TensorPtr> grads = n->backward_fn->apply(g);
            for (size_t k = 0; k < n->inputs.size() && k < grads.size(); ++k) deliver(n->inputs[k], grads[k]);
        }
        pending.erase(pg);
    }
    // the graph is single use: release what this pass visited
    for (Node* n : order) {
        if (n->owner && n->owner->grad_node_.get() == n) {
            NodePtr keep = n->owner->grad_node_;   // `n` must outlive the statements below
            n->owner->grad_node_ = nullptr;
            keep->inputs.clear();
            keep->backward_fn.reset();
        }
    }
    live_.erase(std::remove_if(live_.begin(), live_.end(), [](const std::weak_ptr<Node>& w) { return w.expired(); }), live_.end());
}

}  // namespace autograd
}  // namespace ops
