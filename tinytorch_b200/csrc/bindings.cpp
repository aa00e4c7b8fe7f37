/* pybind11 module `tinytorch_pybind`: the Node class of the reference's
 * Python-facing module (src/bindings.cpp:54-150) over the B200 library.
 *
 * Same class name, method names, keyword arguments and defaults; a NULL from
 * the C ABI becomes ValueError (src/bindings.cpp:22-30); arrays are copied in
 * with tt_fromdata and out through tt_data.  The module links against
 * libtinytorch.so instead of compiling the C sources into itself, so Python
 * and C callers share one device context. */
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <memory>
#include <string>
#include <vector>

#include "autograd.h"
#include "tensor.h"
#include "tt_b200.h"

namespace py = pybind11;
using f32_array = py::array_t<float, py::array::c_style | py::array::forcecast>;

namespace {

[[noreturn]] void fail(const char *what) {
    std::string msg = std::string("tinytorch: ") + what + " failed (invalid arguments or shape mismatch)";
    const char *why = ttb_last_error();
    if (why && *why) msg += std::string(": ") + why;
    throw py::value_error(msg);
}

std::shared_ptr<AGNode> own(AGNode *n, const char *what) {
    if (!n) fail(what);
    return std::shared_ptr<AGNode>(n, [](AGNode *p) { ag_release(p); });
}

py::array_t<float> to_numpy(Tensor *t) {
    if (!t) return py::array_t<float>();
    std::vector<long> dims((size_t)tt_ndim(t));
    tt_shape(t, dims.data());
    std::vector<py::ssize_t> shape(dims.begin(), dims.end());
    py::array_t<float> out(shape);
    const float *src = tt_data(t);
    if (!src) fail("tt_data");
    std::memcpy(out.mutable_data(), src, sizeof(float) * (size_t)tt_numel(t));
    return out;
}

class Node {
public:
    explicit Node(std::shared_ptr<AGNode> n) : n_(std::move(n)) {}

    static Node leaf(f32_array arr, bool requires_grad) {
        py::buffer_info info = arr.request();
        std::vector<long> shape((size_t)info.ndim);
        for (py::ssize_t i = 0; i < info.ndim; i++) shape[(size_t)i] = (long)info.shape[(size_t)i];
        Tensor *t = tt_fromdata(static_cast<const float *>(info.ptr), shape.data(), (int)info.ndim);
        if (!t) fail("tt_fromdata");
        AGNode *n = ag_leaf(t, requires_grad ? 1 : 0);
        tt_release(t);                      /* the node holds its own reference */
        return Node(own(n, "ag_leaf"));
    }

    py::array_t<float> value() const { return to_numpy(ag_value(n_.get())); }

    py::object grad() const {
        Tensor *g = ag_grad(n_.get());
        if (!g) return py::none();
        return to_numpy(g);
    }

    void backward(py::object seed) {
        if (seed.is_none()) { ag_backward(n_.get()); return; }
        f32_array arr = seed.cast<f32_array>();
        py::buffer_info info = arr.request();
        Tensor *v = ag_value(n_.get());
        if (!v || (size_t)info.size != (size_t)tt_numel(v))
            throw py::value_error("tinytorch: seed length mismatch");
        ag_backward_from(n_.get(), static_cast<const float *>(info.ptr), (size_t)info.size);
    }

    Node add(const Node &o) const { return Node(own(ag_add(n_.get(), o.n_.get()), "ag_add")); }
    Node mul(const Node &o) const { return Node(own(ag_mul(n_.get(), o.n_.get()), "ag_mul")); }
    Node addscalar(float s) const { return Node(own(ag_addscalar(n_.get(), s), "ag_addscalar")); }
    Node mulscalar(float s) const { return Node(own(ag_mulscalar(n_.get(), s), "ag_mulscalar")); }
    Node matmul(const Node &o) const { return Node(own(ag_matmul(n_.get(), o.n_.get()), "ag_matmul")); }
    Node relu() const { return Node(own(ag_relu(n_.get()), "ag_relu")); }
    Node softmax() const { return Node(own(ag_softmax(n_.get()), "ag_softmax")); }
    Node padones() const { return Node(own(ag_padones(n_.get()), "ag_padones")); }
    Node reshape(std::vector<long> shape) const {
        return Node(own(ag_reshape(n_.get(), shape.data(), (int)shape.size()), "ag_reshape"));
    }
    Node conv2d(const Node &w, py::object b, int sh, int sw, int ph, int pw) const {
        AGNode *bias = b.is_none() ? nullptr : b.cast<Node>().n_.get();
        return Node(own(ag_conv2d(n_.get(), w.n_.get(), bias, sh, sw, ph, pw), "ag_conv2d"));
    }
    Node maxpool2d(int ph, int pw, int sh, int sw) const {
        return Node(own(ag_maxpool2d(n_.get(), ph, pw, sh, sw), "ag_maxpool2d"));
    }
    Node avgpool2d(int ph, int pw, int sh, int sw) const {
        return Node(own(ag_avgpool2d(n_.get(), ph, pw, sh, sw), "ag_avgpool2d"));
    }

private:
    std::shared_ptr<AGNode> n_;
};

}  // namespace

PYBIND11_MODULE(tinytorch_pybind, m) {
    m.doc() = "tinytorch autograd nodes on the B200 library";
    py::class_<Node>(m, "Node")
        .def_static("leaf", &Node::leaf, py::arg("arr"), py::arg("requires_grad") = true)
        .def("value", &Node::value)
        .def("grad", &Node::grad)
        .def("backward", &Node::backward, py::arg("seed") = py::none())
        .def("add", &Node::add)
        .def("mul", &Node::mul)
        .def("addscalar", &Node::addscalar)
        .def("mulscalar", &Node::mulscalar)
        .def("matmul", &Node::matmul)
        .def("relu", &Node::relu)
        .def("softmax", &Node::softmax)
        .def("padones", &Node::padones)
        .def("reshape", &Node::reshape)
        .def("conv2d", &Node::conv2d, py::arg("w"), py::arg("b") = py::none(), py::arg("stride_h") = 1,
             py::arg("stride_w") = 1, py::arg("pad_h") = 0, py::arg("pad_w") = 0)
        .def("maxpool2d", &Node::maxpool2d, py::arg("pool_h") = 2, py::arg("pool_w") = 2,
             py::arg("stride_h") = 2, py::arg("stride_w") = 2)
        .def("avgpool2d", &Node::avgpool2d, py::arg("pool_h") = 2, py::arg("pool_w") = 2,
             py::arg("stride_h") = 2, py::arg("stride_w") = 2)
        .def("__add__", &Node::add)
        .def("__mul__", &Node::mul);
}
