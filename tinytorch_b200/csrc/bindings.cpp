/* pybind11 module `tinytorch_pybind` over the B200 library.
 *
 * Python surface of the reference's module (src/bindings.cpp:54-150): one class, Node,
 * with the same method names, keyword arguments and defaults, so scripts written for it
 * run unchanged.  A NULL from the C ABI becomes ValueError carrying the library's own
 * error text; arrays go in through tt_fromdata and come out through tt_data.  Unlike the
 * reference's module, which compiles the C sources into itself, this one links against
 * libtinytorch.so, so Python and C callers of one process share one device context.
 *
 * The bindings are a table of lambdas over a handle type; the handle is a shared_ptr whose
 * deleter is ag_release, so Python's garbage collector drives the node reference counts. */
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <memory>
#include <string>
#include <utility>
#include <vector>

#include "autograd.h"
#include "tensor.h"
#include "tt_b200.h"

namespace py = pybind11;

namespace {

using HostArray = py::array_t<float, py::array::c_style | py::array::forcecast>;

/* Python-visible handle of one graph node. */
struct Node {
    std::shared_ptr<AGNode> ref;
    AGNode *raw() const { return ref.get(); }
};

[[noreturn]] void raise_for(const char *call) {
    std::string text = "tinytorch: ";
    text += call;
    text += " failed (invalid arguments or shape mismatch)";
    if (const char *why = ttb_last_error(); why && *why) {
        text += ": ";
        text += why;
    }
    throw py::value_error(text);
}

/* Take ownership of a node the C ABI just returned (one reference), or raise. */
Node adopt(AGNode *fresh, const char *call) {
    if (fresh == nullptr) raise_for(call);
    return Node{std::shared_ptr<AGNode>(fresh, &ag_release)};
}

/* Device tensor -> new NumPy array (waits for the GPU). */
py::array_t<float> export_tensor(Tensor *t) {
    if (t == nullptr) return py::array_t<float>();
    const int rank = tt_ndim(t);
    std::vector<long> extents(static_cast<size_t>(rank));
    tt_shape(t, extents.data());
    py::array_t<float> result(std::vector<py::ssize_t>(extents.begin(), extents.end()));
    const float *host = tt_data(t);
    if (host == nullptr) raise_for("tt_data");
    std::memcpy(result.mutable_data(), host, sizeof(float) * static_cast<size_t>(tt_numel(t)));
    return result;
}

/* NumPy array -> leaf node. */
Node import_leaf(HostArray values, bool requires_grad) {
    const py::buffer_info view = values.request();
    std::vector<long> extents;
    extents.reserve(static_cast<size_t>(view.ndim));
    for (py::ssize_t extent : view.shape) extents.push_back(static_cast<long>(extent));
    Tensor *payload = tt_fromdata(static_cast<const float *>(view.ptr), extents.data(), static_cast<int>(extents.size()));
    if (payload == nullptr) raise_for("tt_fromdata");
    AGNode *leaf = ag_leaf(payload, requires_grad ? 1 : 0);
    tt_release(payload);                    /* the node holds its own reference */
    return adopt(leaf, "ag_leaf");
}

/* Reverse pass from ones, or from a seed array of exactly the root's size. */
void run_backward(const Node &root, const py::object &seed) {
    if (seed.is_none()) {
        ag_backward(root.raw());
        return;
    }
    const HostArray values = seed.cast<HostArray>();
    const py::buffer_info view = values.request();
    const Tensor *value = ag_value(root.raw());
    if (value == nullptr || static_cast<long>(view.size) != tt_numel(value))
        throw py::value_error("tinytorch: seed length mismatch");
    ag_backward_from(root.raw(), static_cast<const float *>(view.ptr), static_cast<size_t>(view.size));
}

/* Binders for the three call shapes most builders have. */
template <AGNode *(*Build)(AGNode *)>
auto unary(const char *call) {
    return [call](const Node &x) { return adopt(Build(x.raw()), call); };
}
template <AGNode *(*Build)(AGNode *, AGNode *)>
auto binary(const char *call) {
    return [call](const Node &x, const Node &y) { return adopt(Build(x.raw(), y.raw()), call); };
}
template <AGNode *(*Build)(AGNode *, float)>
auto with_scalar(const char *call) {
    return [call](const Node &x, float c) { return adopt(Build(x.raw(), c), call); };
}
template <AGNode *(*Build)(AGNode *, int, int, int, int)>
auto pooling(const char *call) {
    return [call](const Node &x, int window_h, int window_w, int stride_h, int stride_w) {
        return adopt(Build(x.raw(), window_h, window_w, stride_h, stride_w), call);
    };
}

}  // namespace

PYBIND11_MODULE(tinytorch_pybind, m) {
    m.doc() = "tinytorch autograd nodes on the B200 library";
    using namespace pybind11::literals;

    py::class_<Node> node(m, "Node");
    node.def_static("leaf", &import_leaf, "arr"_a, "requires_grad"_a = true);

    /* what the node holds */
    node.def("value", [](const Node &x) { return export_tensor(ag_value(x.raw())); });
    node.def("grad", [](const Node &x) -> py::object {
        Tensor *g = ag_grad(x.raw());
        if (g == nullptr) return py::none();
        return export_tensor(g);
    });
    node.def("backward", &run_backward, "seed"_a = py::none());

    /* builders */
    node.def("add", binary<&ag_add>("ag_add"));
    node.def("mul", binary<&ag_mul>("ag_mul"));
    node.def("__add__", binary<&ag_add>("ag_add"));
    node.def("__mul__", binary<&ag_mul>("ag_mul"));
    node.def("matmul", binary<&ag_matmul>("ag_matmul"));
    node.def("addscalar", with_scalar<&ag_addscalar>("ag_addscalar"));
    node.def("mulscalar", with_scalar<&ag_mulscalar>("ag_mulscalar"));
    node.def("relu", unary<&ag_relu>("ag_relu"));
    node.def("softmax", unary<&ag_softmax>("ag_softmax"));
    node.def("padones", unary<&ag_padones>("ag_padones"));
    node.def("reshape", [](const Node &x, std::vector<long> extents) {
        return adopt(ag_reshape(x.raw(), extents.data(), static_cast<int>(extents.size())), "ag_reshape");
    });
    node.def("conv2d",
             [](const Node &x, const Node &filters, const py::object &bias, int stride_h, int stride_w, int pad_h, int pad_w) {
                 AGNode *b = bias.is_none() ? nullptr : bias.cast<const Node &>().raw();
                 return adopt(ag_conv2d(x.raw(), filters.raw(), b, stride_h, stride_w, pad_h, pad_w), "ag_conv2d");
             },
             "w"_a, "b"_a = py::none(), "stride_h"_a = 1, "stride_w"_a = 1, "pad_h"_a = 0, "pad_w"_a = 0);
    node.def("maxpool2d", pooling<&ag_maxpool2d>("ag_maxpool2d"), "pool_h"_a = 2, "pool_w"_a = 2, "stride_h"_a = 2,
             "stride_w"_a = 2);
    node.def("avgpool2d", pooling<&ag_avgpool2d>("ag_avgpool2d"), "pool_h"_a = 2, "pool_w"_a = 2, "stride_h"_a = 2,
             "stride_w"_a = 2);
}
