// Backward-function interface of the autograd engine.  Each ops:: function that
// records a node supplies one of these; the concrete classes live next to the
// operators that create them (ops.cpp, lm_loss.cpp).
#pragma once
#include <functional>
#include <memory>
#include <vector>

#include "tensor.h"

namespace ops {

class BackwardFunction {
public:
    virtual ~BackwardFunction() = default;
    // grad_output -> one gradient per recorded input (nullptr where none is due)
    virtual std::vector<TensorPtr> apply(const TensorPtr& grad_output) = 0;
};
using BackwardFunctionPtr = std::shared_ptr<BackwardFunction>;

// Adapter used by most operators: the backward rule is a closure over what it needs.
class ClosureBackward : public BackwardFunction {
public:
    using Fn = std::function<std::vector<TensorPtr>(const TensorPtr&)>;
    explicit ClosureBackward(Fn fn) : fn_(std::move(fn)) {}
    std::vector<TensorPtr> apply(const TensorPtr& g) override { return fn_(g); }
private:
    Fn fn_;
};

}  // namespace ops
