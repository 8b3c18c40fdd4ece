// Reverse-mode autograd for ops::Tensor.
//
// Same entry points as the reference's core/autograd_engine.h
// (Engine::instance(), register_node, run_backward, clear_graph, set_enabled),
// different bookkeeping: a node hangs off the tensor it produced and keeps its
// input tensors alive, so there is no process-wide tensor map; run_backward
// walks the nodes reachable from the roots in reverse topological order,
// accumulates gradients out of place (no shared-buffer aliasing), adds into
// leaf .grad across calls, and releases the visited graph afterwards.
#pragma once
#include <memory>
#include <vector>

#include "backward_functions.h"
#include "tensor.h"

namespace ops {
namespace autograd {

class Node {
public:
    Tensor* owner = nullptr;                 // the tensor this node produced (kept alive by its consumers / the caller)
    std::vector<TensorPtr> inputs;           // recorded inputs, in backward-function order
    BackwardFunctionPtr backward_fn;
    TensorPtr tensor;                        // set only while a backward pass runs (API compatibility)
};
using NodePtr = std::shared_ptr<Node>;

class Engine {
public:
    static Engine& instance();
    void run_backward(const std::vector<TensorPtr>& outputs, const std::vector<TensorPtr>& output_grads = {});
    NodePtr register_node(const TensorPtr& output, const std::vector<TensorPtr>& inputs, BackwardFunctionPtr backward_fn);
    NodePtr get_node(const TensorPtr& tensor);
    void clear_graph();
    void set_enabled(bool enabled) { enabled_ = enabled; }
    bool is_enabled() const { return enabled_; }

private:
    Engine() = default;
    bool enabled_ = true;
    std::vector<std::weak_ptr<Node>> live_;   // nodes recorded since the last clear_graph()
};

// RAII: no nodes are recorded while one of these is alive.
class NoGradGuard {
public:
    NoGradGuard() : prev_(Engine::instance().is_enabled()) { Engine::instance().set_enabled(false); }
    ~NoGradGuard() { Engine::instance().set_enabled(prev_); }
private:
    bool prev_;
};

}  // namespace autograd
}  // namespace ops
