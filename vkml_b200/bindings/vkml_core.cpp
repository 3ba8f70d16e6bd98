// Python extension `_vkml_core` for vkML with the B200 backend behind it.
//
// vkML's Python package (python/vkml/__init__.py, nn.py, optim.py ...) imports one native
// module, `_vkml_core`, and reads every name it needs from it (python/vkml/__init__.py:15-239).
// The reference builds that module with nanobind (bindings/module.cpp:235-1014).  This file
// provides the same module -- same names, same argument names and defaults, same exception
// mapping -- with pybind11, and with the device slot vkML calls "vulkan" served by the B200
// adapter: `init_vulkan(i)` registers vkml_b200::B200Backend under Device::vulkan(i), so
// `V.best_device()`, `V.nn`, `V.optim`, `Tensor.backward()` and `.numpy()` drive the CUDA
// backend with no change to the Python package.
//
// The `vulkan_*` diagnostics the package re-exports (python/vkml/__init__.py:188-239) are
// answered from the C ABI: device reports from b200_get_caps, counters from b200_get_stats,
// per-dispatch times from b200_profile_read.
//
// Everything above the backend interface is vkML's own code, compiled from its sources; this
// file only translates Python calls into calls of vkML's public C++ API.
#include <pybind11/functional.h>
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "b200_backend.h"
#include "vkml_b200.h"

#include "vkml/api/ops.h"
#include "vkml/api/tensor.h"
#include "vkml/autograd/autograd.h"
#include "vkml/backend/api/backend.h"
#include "vkml/dispatch/executor.h"
#include "vkml/graph/grad_mode.h"
#include "vkml/graph/op.h"
#include "vkml/util/coverage.h"
#include "vkml/util/decisions.h"
#include "vkml/util/env.h"
#include "vkml/util/error.h"
#include "vkml/util/log.h"

#include <array>
#include <cstring>
#include <deque>
#include <map>
#include <mutex>
#include <optional>
#include <string>
#include <vector>

namespace py = pybind11;
using namespace pybind11::literals;
using vkml::Device;
using vkml::DType;
using vkml::Tensor;

namespace {

using Dims = std::vector<int64_t>;
using Pair = std::array<int, 2>;

// ---------------------------------------------------------------------------
// numpy <-> Tensor
// ---------------------------------------------------------------------------

DType dtype_of(const py::dtype& dt) {
    const char kind = dt.kind();
    const auto size = dt.itemsize();
    if (kind == 'f' && size == 4) return DType::F32;
    if (kind == 'f' && size == 2) return DType::F16;
    if (kind == 'i' && size == 4) return DType::I32;
    if (kind == 'i' && size == 8) return DType::I64;
    if (kind == 'b') return DType::Bool;
    throw vkml::DTypeError("unsupported array dtype; vkml handles f32, f16, i32, i64 and bool");
}

py::dtype numpy_dtype(DType dt) {
    switch (dt) {
        case DType::F32: return py::dtype("float32");
        case DType::F16: return py::dtype("float16");
        case DType::I32: return py::dtype("int32");
        case DType::I64: return py::dtype("int64");
        case DType::Bool: return py::dtype("bool");
    }
    throw vkml::DTypeError("unknown dtype");
}

// A C-contiguous host array becomes a tensor on `device` (one upload), optionally cast.
Tensor tensor_from_array(const py::array& array, std::optional<DType> want, Device device) {
    if (!(array.flags() & py::array::c_style)) {
        throw vkml::ShapeError("from_numpy expects a C-contiguous array");
    }
    Dims dims(array.shape(), array.shape() + array.ndim());
    const DType have = dtype_of(array.dtype());
    Tensor t = Tensor::from_host(array.data(), dims, have, device);
    return (want && *want != have) ? t.to(*want) : t;
}

// Always a copy into memory numpy owns: the tensor may be a strided view, may live on the device
// and may not have been evaluated yet.
py::array tensor_to_numpy(const Tensor& t) {
    const Tensor dense = t.contiguous();
    dense.realize();
    const Dims shape = dense.shape();
    py::array out(numpy_dtype(dense.dtype()), std::vector<py::ssize_t>(shape.begin(), shape.end()));
    if (dense.numel() > 0) {
        dense.to_host(out.mutable_data());
    }
    return out;
}

std::vector<int> axes_of(const py::object& dim) {
    std::vector<int> axes;
    if (dim.is_none()) return axes;
    if (py::isinstance<py::int_>(dim)) {
        axes.push_back(dim.cast<int>());
        return axes;
    }
    for (py::handle h : dim) axes.push_back(h.cast<int>());
    return axes;
}

// x[i], x[a:b:c], x[None] and tuples of those (numpy's basic indexing; no index arrays).
Tensor index_tensor(const Tensor& self, const py::object& key) {
    py::tuple items = py::isinstance<py::tuple>(key) ? key.cast<py::tuple>() : py::make_tuple(key);
    int consumed = 0;
    for (py::handle h : items) consumed += h.is_none() ? 0 : 1;
    if (consumed > self.ndim()) {
        throw vkml::IndexError("too many indices for tensor of rank " + std::to_string(self.ndim()));
    }
    Tensor out = self;
    int axis = 0;
    for (py::handle h : items) {
        if (h.is_none()) {
            out = out.unsqueeze(axis++);
        } else if (py::isinstance<py::slice>(h)) {
            py::ssize_t start = 0, stop = 0, step = 0, len = 0;
            if (!h.cast<py::slice>().compute(out.size(axis), &start, &stop, &step, &len)) {
                throw py::error_already_set();
            }
            if (step <= 0) throw vkml::IndexError("negative or zero slice steps are not supported");
            out = out.slice(axis++, start, stop, step);
        } else if (py::isinstance<py::int_>(h)) {
            const int64_t extent = out.size(axis);
            const int64_t given = h.cast<int64_t>();
            const int64_t i = given < 0 ? given + extent : given;
            if (i < 0 || i >= extent) {
                throw vkml::IndexError("index " + std::to_string(given) + " is out of range for axis " +
                                       std::to_string(axis) + " with extent " + std::to_string(extent));
            }
            out = out.slice(axis, i, i + 1).squeeze(axis);  // the axis is gone: the next index lands here
        } else {
            throw vkml::IndexError("unsupported index type; vkml supports integers, slices and None "
                                   "(advanced indexing is not implemented)");
        }
    }
    return out;
}

// ---------------------------------------------------------------------------
// the B200 behind vkML's "vulkan" device slot
// ---------------------------------------------------------------------------

int cuda_device_count() {
    int n = 0;
    return b200_device_count(&n) == B200_OK ? n : 0;
}

// Capabilities of every CUDA device, read through short-lived contexts the first time they are
// asked for (a report must not need the backend to be registered).
const std::vector<b200_caps>& device_caps() {
    static std::mutex mu;
    static std::vector<b200_caps> caps;
    static bool probed = false;
    const std::lock_guard<std::mutex> lock(mu);
    if (!probed) {
        probed = true;
        for (int i = 0, n = cuda_device_count(); i < n; ++i) {
            b200_caps c{};
            b200_ctx* ctx = nullptr;
            if (b200_create(i, &ctx) == B200_OK) {
                b200_get_caps(ctx, &c);
                b200_destroy(ctx);
            }
            caps.push_back(c);
        }
    }
    return caps;
}

std::string unavailable_reason() {
    int n = 0;
    if (b200_device_count(&n) != B200_OK) return "the CUDA driver reported no usable device";
    if (n == 0) return "no CUDA device is visible to this process";
    return "";
}

vkml_b200::B200Backend& device_backend(int index) {
    if (index < 0 || index >= cuda_device_count()) {
        throw vkml::DeviceError("no device with index " + std::to_string(index) + " (" +
                                std::to_string(cuda_device_count()) + " visible)");
    }
    return vkml_b200::b200_backend(index);
}

// Device times per dispatch, grouped by submission (= one Backend::compute call), as vkML's
// profiling hooks present them (bindings/module.cpp:222-230, python/vkml/attribution.py:263-365):
// every submission is a run of dispatch records followed by one "submit" record for the whole
// window.  The launches of a context run serially on one stream, so a dispatch starts where its
// predecessor ended and the window is the sum.
struct ProfileRecord {
    std::string label;
    double gpu_ms = 0.0, start_ms = 0.0;
    uint64_t submission = 0;
    uint64_t dispatch = 0;
};
struct ProfileStore {
    std::vector<ProfileRecord> last;                   // the most recent submission
    std::deque<std::vector<ProfileRecord>> history;    // the last `keep` submissions, oldest first
    size_t keep = 0;
    uint64_t resolved = 0;                             // submissions seen, including those dropped
};
std::map<int, ProfileStore>& profile_stores() {
    static auto* stores = new std::map<int, ProfileStore>();
    return *stores;
}

ProfileStore& read_profile(int index) {
    b200_ctx* ctx = device_backend(index).context();
    ProfileStore& store = profile_stores()[index];
    std::vector<b200_profile_record> records(1 << 16);
    size_t n = 0;
    if (b200_profile_read(ctx, records.data(), records.size(), &n) != B200_OK) {
        throw vkml::DeviceError(std::string("profile read failed: ") + b200_last_error(ctx));
    }
    size_t i = 0;
    while (i < n) {
        std::vector<ProfileRecord> group;
        const uint32_t submission = records[i].submission;
        double at = 0.0;
        for (; i < n && records[i].submission == submission; ++i) {
            const double ms = records[i].ms > 0.0F ? records[i].ms : 0.0;
            group.push_back({records[i].label, ms, at, submission, static_cast<uint64_t>(group.size() + 1)});
            at += ms;
        }
        group.push_back({"submit", at, 0.0, submission, 0});
        if (store.keep > 0) {
            ++store.resolved;  // offered to the retention window, whether or not it is still held
            store.history.push_back(group);
            while (store.history.size() > store.keep) store.history.pop_front();
        }
        store.last = std::move(group);
    }
    return store;
}

py::dict record_dict(const ProfileRecord& r) {
    py::dict e;
    e["label"] = r.label;
    e["gpu_ms"] = r.gpu_ms;
    e["start_ms"] = r.start_ms;
    e["submission"] = r.submission;
    e["dispatch"] = r.dispatch;
    return e;
}

}  // namespace

PYBIND11_MODULE(_vkml_core, m) {
    m.doc() = "vkML core with the B200 (sm_100a) backend behind the vulkan device slot";
    m.attr("__version__") = "0.1.0";

    // -- errors: vkML's exception types, each on the Python base the package and its tests expect
    //    (bindings/module.cpp:243-250).  pybind11 tries translators last-registered first, so the
    //    base class goes in first and the derived classes are matched before it.
    py::register_exception<vkml::Error>(m, "Error", PyExc_RuntimeError);
    py::register_exception<vkml::InternalError>(m, "InternalError", PyExc_RuntimeError);
    py::register_exception<vkml::NotImplementedError>(m, "NotImplementedError", PyExc_NotImplementedError);
    py::register_exception<vkml::OutOfMemoryError>(m, "OutOfMemoryError", PyExc_MemoryError);
    py::register_exception<vkml::DeviceError>(m, "DeviceError", PyExc_RuntimeError);
    py::register_exception<vkml::IndexError>(m, "IndexError", PyExc_IndexError);
    py::register_exception<vkml::DTypeError>(m, "DTypeError", PyExc_TypeError);
    py::register_exception<vkml::ShapeError>(m, "ShapeError", PyExc_ValueError);

    // -- logging, dtypes, devices, execution mode
    py::enum_<vkml::LogLevel>(m, "LogLevel")
        .value("TRACE", vkml::LogLevel::Trace)
        .value("DEBUG", vkml::LogLevel::Debug)
        .value("INFO", vkml::LogLevel::Info)
        .value("WARN", vkml::LogLevel::Warn)
        .value("ERROR", vkml::LogLevel::Error)
        .value("OFF", vkml::LogLevel::Off);
    m.def("set_log_level", &vkml::set_log_level, "level"_a);
    m.def("log_level", &vkml::log_level);
    m.def(
        "set_log_callback",
        [](std::optional<std::function<void(vkml::LogLevel, std::string)>> fn) {
            if (!fn || !*fn) {
                vkml::set_log_callback(nullptr);
                return;
            }
            vkml::set_log_callback([fn = std::move(*fn)](vkml::LogLevel level, std::string_view text) {
                const py::gil_scoped_acquire gil;
                fn(level, std::string(text));
            });
        },
        "callback"_a.none(true));

    py::enum_<DType>(m, "dtype")
        .value("float32", DType::F32)
        .value("float16", DType::F16)
        .value("int32", DType::I32)
        .value("int64", DType::I64)
        .value("bool", DType::Bool);
    m.def("dtype_size", &vkml::dtype_size, "dtype"_a);
    m.def("dtype_name", [](DType d) { return std::string(vkml::dtype_name(d)); }, "dtype"_a);

    py::class_<Device>(m, "device")
        .def(py::init<>())
        .def(py::init([](const std::string& spec) { return Device::parse(spec); }), "spec"_a)
        .def_property_readonly("index", &Device::index)
        .def_property_readonly("is_cpu", &Device::is_cpu)
        .def("__repr__", [](const Device& d) { return "device('" + d.str() + "')"; })
        .def("__str__", &Device::str)
        .def("__eq__", [](const Device& a, const Device& b) { return a == b; }, py::is_operator())
        .def("__hash__", [](const Device& d) {
            return static_cast<size_t>(d.index()) * 31U + static_cast<size_t>(d.kind());
        });
    m.def("cpu_device", &Device::cpu);
    m.def("available_devices", &vkml::available_devices);
    m.def("set_eager", &vkml::set_eager, "enabled"_a);
    m.def("is_eager", &vkml::eager);

    m.def("_coverage_enabled", &vkml::coverage::enabled);
    m.def("_coverage_dump", &vkml::coverage::dump, "path"_a);
    m.def("_coverage_clear", &vkml::coverage::clear);
    m.def("_op_names", [] {
        std::vector<std::string> names;
        for (int i = 0; i < vkml::kNumOps; ++i) names.emplace_back(vkml::op_name(static_cast<vkml::OpKind>(i)));
        return names;
    });
    m.def("_op_categories", [] {
        std::vector<std::pair<std::string, std::string>> out;
        for (int i = 0; i < vkml::kNumOps; ++i) {
            const auto op = static_cast<vkml::OpKind>(i);
            out.emplace_back(vkml::op_name(op), vkml::is_leaf_op(op) ? "leaf" : vkml::is_view_op(op) ? "view" : "compute");
        }
        return out;
    });

    // -- Tensor
    py::class_<Tensor> tensor(m, "Tensor");
    tensor.def(py::init<>())
        .def_property_readonly("shape", [](const Tensor& t) { return py::tuple(py::cast(t.shape())); })
        .def_property_readonly("ndim", &Tensor::ndim)
        .def_property_readonly("size", &Tensor::numel)
        .def_property_readonly("dtype", &Tensor::dtype)
        .def_property_readonly("device", &Tensor::device)
        .def_property_readonly("strides", &Tensor::strides)  // bytes, as in numpy
        .def_property_readonly("is_contiguous", &Tensor::is_contiguous)
        .def_property_readonly("T", [](const Tensor& t) { return t.transpose(-2, -1); })
        .def("defined", &Tensor::defined)
        .def("__bool__", &Tensor::defined)
        .def("__len__",
             [](const Tensor& t) {
                 if (t.ndim() == 0) throw vkml::IndexError("len() of a 0-dimensional tensor");
                 return t.size(0);
             })
        .def("__repr__", &Tensor::str)
        .def("__str__", &Tensor::str)
        .def("realize",
             [](const Tensor& t) {
                 t.realize();
                 return t;
             })
        .def("item", &Tensor::item)
        .def("numpy", &tensor_to_numpy)
        .def("__array__", [](const Tensor& t, const py::args&, const py::kwargs&) { return tensor_to_numpy(t); })
        .def("reshape", [](const Tensor& t, const Dims& d) { return t.reshape(d); }, "shape"_a)
        .def("view", [](const Tensor& t, const Dims& d) { return t.reshape(d); }, "shape"_a)
        .def("permute", [](const Tensor& t, const std::vector<int>& p) { return t.permute(p); }, "dims"_a)
        .def("transpose", &Tensor::transpose, "dim0"_a, "dim1"_a)
        .def("squeeze", &Tensor::squeeze, "dim"_a)
        .def("unsqueeze", &Tensor::unsqueeze, "dim"_a)
        .def("broadcast_to", [](const Tensor& t, const Dims& d) { return t.broadcast_to(d); }, "shape"_a)
        .def("contiguous", &Tensor::contiguous)
        .def("to", &Tensor::to, "dtype"_a)
        .def("astype", &Tensor::to, "dtype"_a)
        .def("__getitem__", &index_tensor, "key"_a)
        .def_property("requires_grad", &Tensor::requires_grad, [](Tensor& t, bool v) { t.set_requires_grad(v); })
        .def_property("grad", &Tensor::grad, [](Tensor& t, const Tensor& g) { t.set_grad(g); })
        .def("backward", [](const Tensor& t) { vkml::backward(t); })
        .def("assign_", &Tensor::assign_, "src"_a)
        .def("detach", [](const Tensor& t) { return vkml::detach(t); });

    // operators
    tensor.def("__add__", [](const Tensor& a, const Tensor& b) { return a + b; }, py::is_operator())
        .def("__add__", [](const Tensor& a, double s) { return a + s; }, py::is_operator())
        .def("__radd__", [](const Tensor& a, double s) { return a + s; }, py::is_operator())
        .def("__sub__", [](const Tensor& a, const Tensor& b) { return a - b; }, py::is_operator())
        .def("__sub__", [](const Tensor& a, double s) { return a - s; }, py::is_operator())
        .def("__rsub__", [](const Tensor& a, double s) { return vkml::add(vkml::neg(a), s); }, py::is_operator())
        .def("__mul__", [](const Tensor& a, const Tensor& b) { return a * b; }, py::is_operator())
        .def("__mul__", [](const Tensor& a, double s) { return a * s; }, py::is_operator())
        .def("__rmul__", [](const Tensor& a, double s) { return a * s; }, py::is_operator())
        .def("__truediv__", [](const Tensor& a, const Tensor& b) { return a / b; }, py::is_operator())
        .def("__truediv__", [](const Tensor& a, double s) { return a / s; }, py::is_operator())
        .def("__rtruediv__", [](const Tensor& a, double s) { return vkml::mul(vkml::reciprocal(a), s); },
             py::is_operator())
        .def("__pow__", [](const Tensor& a, double s) { return vkml::pow(a, s); }, py::is_operator())
        .def("__neg__", [](const Tensor& a) { return -a; }, py::is_operator())
        .def("__matmul__", [](const Tensor& a, const Tensor& b) { return vkml::matmul(a, b); }, py::is_operator())
        .def("__lt__", [](const Tensor& a, const Tensor& b) { return vkml::less(a, b); }, py::is_operator())
        .def("__gt__", [](const Tensor& a, const Tensor& b) { return vkml::greater(a, b); }, py::is_operator())
        .def("__le__", [](const Tensor& a, const Tensor& b) { return vkml::less_equal(a, b); }, py::is_operator())
        .def("__ge__", [](const Tensor& a, const Tensor& b) { return vkml::greater_equal(a, b); }, py::is_operator());
    tensor.attr("__hash__") = py::none();  // comparison operators build tensors, so identity hashing would mislead

    // One table per call shape: every entry becomes a module function, the marked ones also a
    // Tensor method (`x.relu()`), so the two spellings can never drift apart.
    using Unary = Tensor (*)(const Tensor&);
    struct UnaryEntry {
        const char* name;
        Unary fn;
        bool method;
    };
    const UnaryEntry unary[] = {
        {"neg", &vkml::neg, false},         {"abs", &vkml::abs, true},       {"sign", &vkml::sign, false},
        {"square", &vkml::square, false},   {"sqrt", &vkml::sqrt, true},     {"rsqrt", &vkml::rsqrt, false},
        {"reciprocal", &vkml::reciprocal, false}, {"exp", &vkml::exp, true}, {"log", &vkml::log, true},
        {"erf", &vkml::erf, false},         {"erfc", &vkml::erfc, false},    {"sin", &vkml::sin, false},
        {"cos", &vkml::cos, false},         {"tanh", &vkml::tanh, true},     {"sigmoid", &vkml::sigmoid, true},
        {"relu", &vkml::relu, true},        {"gelu", &vkml::gelu, true},     {"silu", &vkml::silu, true},
        {"zeros_like", &vkml::zeros_like, false}, {"ones_like", &vkml::ones_like, false},
        {"detach", &vkml::detach, false},
    };
    for (const UnaryEntry& e : unary) {
        m.def(e.name, e.fn, "input"_a);
        if (e.method) tensor.def(e.name, e.fn);
    }
    using Binary = Tensor (*)(const Tensor&, const Tensor&);
    const std::pair<const char*, Binary> binary[] = {
        {"add", &vkml::add},         {"sub", &vkml::sub},         {"mul", &vkml::mul},
        {"div", &vkml::div},         {"pow", &vkml::pow},         {"maximum", &vkml::maximum},
        {"minimum", &vkml::minimum}, {"equal", &vkml::equal},     {"less", &vkml::less},
        {"greater", &vkml::greater}, {"less_equal", &vkml::less_equal}, {"greater_equal", &vkml::greater_equal},
        {"not_equal", &vkml::not_equal}, {"matmul", &vkml::matmul},
    };
    for (const auto& [name, fn] : binary) m.def(name, fn, "a"_a, "b"_a);
    using Scalar = Tensor (*)(const Tensor&, double);
    const std::pair<const char*, Scalar> scalar[] = {
        {"add", &vkml::add}, {"sub", &vkml::sub}, {"mul", &vkml::mul}, {"div", &vkml::div}, {"pow", &vkml::pow}};
    for (const auto& [name, fn] : scalar) m.def(name, fn, "a"_a, "s"_a);  // overloads of the tensor forms
    tensor.def("matmul", &vkml::matmul, "other"_a);

    using Reduce = Tensor (*)(const Tensor&, std::span<const int>, bool);
    struct ReduceEntry {
        const char* function;
        const char* method;  // nullptr: no method form
        Reduce fn;
    };
    const ReduceEntry reductions[] = {{"sum", "sum", &vkml::sum},   {"mean", "mean", &vkml::mean},
                                      {"prod", nullptr, &vkml::prod}, {"amax", "max", &vkml::max},
                                      {"amin", "min", &vkml::min}};
    for (const ReduceEntry& e : reductions) {
        const Reduce fn = e.fn;
        auto call = [fn](const Tensor& t, const py::object& dim, bool keepdim) { return fn(t, axes_of(dim), keepdim); };
        m.def(e.function, call, "input"_a, "dim"_a = py::none(), "keepdim"_a = false);
        if (e.method != nullptr) tensor.def(e.method, call, "dim"_a = py::none(), "keepdim"_a = false);
    }
    m.def("argmax", &vkml::argmax, "input"_a, "dim"_a, "keepdim"_a = false);
    m.def("argmin", &vkml::argmin, "input"_a, "dim"_a, "keepdim"_a = false);
    m.def("softmax", &vkml::softmax, "input"_a, "dim"_a = -1);
    m.def("log_softmax", &vkml::log_softmax, "input"_a, "dim"_a = -1);
    tensor.def("softmax", &vkml::softmax, "dim"_a = -1).def("log_softmax", &vkml::log_softmax, "dim"_a = -1);

    // -- construction
    m.def("from_numpy", &tensor_from_array, "array"_a, "dtype"_a = py::none(), "device"_a = Device::cpu());
    m.def("zeros", [](const Dims& d, DType dt, Device dev) { return Tensor::zeros(d, dt, dev); }, "shape"_a,
          "dtype"_a = DType::F32, "device"_a = Device::cpu());
    m.def("ones", [](const Dims& d, DType dt, Device dev) { return Tensor::ones(d, dt, dev); }, "shape"_a,
          "dtype"_a = DType::F32, "device"_a = Device::cpu());
    m.def("full", [](const Dims& d, double v, DType dt, Device dev) { return Tensor::full(d, v, dt, dev); },
          "shape"_a, "value"_a, "dtype"_a = DType::F32, "device"_a = Device::cpu());
    m.def("full_like", &vkml::full_like, "input"_a, "value"_a);
    m.def("arange", &Tensor::arange, "start"_a, "stop"_a, "step"_a = 1.0, "dtype"_a = DType::F32,
          "device"_a = Device::cpu());
    m.def("rand", [](const Dims& d, uint64_t seed, uint64_t offset, Device dev) { return vkml::rand(d, seed, offset, dev); },
          "shape"_a, "seed"_a, "offset"_a = 0, "device"_a = Device::cpu());

    // -- the remaining operators
    m.def("scaled_add", &vkml::scaled_add, "a"_a, "b"_a, "alpha"_a, "beta"_a);
    m.def("clamp", &vkml::clamp, "input"_a, "min"_a, "max"_a);
    m.def("clamp_min", &vkml::clamp_min, "input"_a, "min"_a);
    m.def("clamp_max", &vkml::clamp_max, "input"_a, "max"_a);
    m.def("where", &vkml::where, "condition"_a, "x"_a, "y"_a);
    m.def("cat", [](const std::vector<Tensor>& ts, int axis) { return vkml::cat(ts, axis); }, "tensors"_a, "axis"_a = 0);
    m.def("masked_fill", &vkml::masked_fill, "input"_a, "mask"_a, "value"_a);
    m.def("triu", &vkml::triu, "input"_a, "diagonal"_a = 0);
    m.def("tril", &vkml::tril, "input"_a, "diagonal"_a = 0);
    m.def("index_select", &vkml::index_select, "input"_a, "axis"_a, "index"_a);
    m.def("scatter_add", &vkml::scatter_add, "src"_a, "axis"_a, "index"_a, "dim_size"_a);
    m.def("layer_norm", &vkml::layer_norm, "input"_a, "normalized_axes"_a = 1, "eps"_a = 1e-5);
    m.def("rms_norm", &vkml::rms_norm, "input"_a, "normalized_axes"_a = 1, "eps"_a = 1e-5);
    m.def("dropout", &vkml::dropout, "input"_a, "p"_a, "seed"_a, "offset"_a = 0, "training"_a = true);
    m.def("batch_norm", &vkml::batch_norm, "input"_a, "mean"_a, "variance"_a, "weight"_a = Tensor{},
          "bias"_a = Tensor{}, "eps"_a = 1e-5);

    const Pair unit{1, 1}, none{0, 0};
    m.def("conv2d", &vkml::conv2d, "input"_a, "weight"_a, "bias"_a = Tensor{}, "stride"_a = unit, "padding"_a = none,
          "dilation"_a = unit);
    m.def("im2col", &vkml::im2col, "input"_a, "kernel"_a, "stride"_a = unit, "padding"_a = none, "dilation"_a = unit);
    m.def("col2im", &vkml::col2im, "cols"_a, "image"_a, "kernel"_a, "stride"_a = unit, "padding"_a = none,
          "dilation"_a = unit);
    m.def("max_pool2d", &vkml::max_pool2d, "input"_a, "kernel"_a, "stride"_a = none, "padding"_a = none,
          "dilation"_a = unit);
    m.def("avg_pool2d", &vkml::avg_pool2d, "input"_a, "kernel"_a, "stride"_a = none, "padding"_a = none);

    py::enum_<vkml::Reduction>(m, "Reduction")
        .value("mean", vkml::Reduction::Mean)
        .value("sum", vkml::Reduction::Sum)
        .value("none", vkml::Reduction::None);
    const auto mean = vkml::Reduction::Mean;
    m.def("mse_loss", &vkml::mse_loss, "input"_a, "target"_a, "reduction"_a = mean);
    m.def("cross_entropy", &vkml::cross_entropy, "logits"_a, "target"_a, "reduction"_a = mean);
    m.def("binary_cross_entropy_with_logits", &vkml::binary_cross_entropy_with_logits, "logits"_a, "target"_a,
          "reduction"_a = mean);
    m.def("kl_div", &vkml::kl_div, "input"_a, "target"_a, "reduction"_a = mean, "log_target"_a = false);
    m.def("huber_loss", &vkml::huber_loss, "input"_a, "target"_a, "reduction"_a = mean, "delta"_a = 1.0);

    // -- evaluation, assignment, autograd
    m.def(
        "realize",
        [](const std::vector<Tensor>& tensors) {
            std::vector<vkml::NodePtr> roots;
            for (const Tensor& t : tensors) {
                // the scheduler skips a null root silently: the call would look like a success
                if (!t.defined()) throw vkml::Error("realize() on an undefined tensor");
                roots.push_back(t.node());
            }
            vkml::realize(roots);
        },
        "tensors"_a);
    m.def("assign", [](const std::vector<Tensor>& dst, const std::vector<Tensor>& src) { vkml::assign(dst, src); },
          "destinations"_a, "sources"_a);
    m.def("backward", [](const Tensor& t) { vkml::backward(t); }, "tensor"_a);
    m.def("backward", [](const Tensor& t, const Tensor& g) { vkml::backward(t, g); }, "tensor"_a, "gradient"_a);
    m.def("set_grad_enabled", &vkml::set_grad_enabled, "enabled"_a);
    m.def("is_grad_enabled", &vkml::grad_enabled);

    // -- observability (published from any layer: not tied to a device)
    m.def("configuration", [] {
        py::list out;
        for (const vkml::ObservedSwitch& s : vkml::observed_environment()) {
            out.append(py::dict("name"_a = s.name, "value"_a = s.value, "set"_a = s.set));
        }
        return out;
    });
    m.def("record_decisions", [](size_t capacity) { vkml::observe::start_recording(capacity); }, "capacity"_a = 256);
    m.def("stop_recording_decisions", [] { vkml::observe::stop_recording(); });
    m.def("decisions", [] {
        py::list out;
        for (const vkml::observe::RecordedDecision& d : vkml::observe::recorded()) {
            out.append(py::dict("site"_a = d.site, "op"_a = d.op, "chose"_a = d.chose, "instead_of"_a = d.instead_of,
                                "because"_a = d.because, "required"_a = d.required, "available"_a = d.available,
                                "seq"_a = d.seq, "dispatch"_a = d.dispatch));
        }
        return out;
    });
    m.def("decisions_published", [] { return vkml::observe::published(); });

    // -- the device slot vkML calls "vulkan", served by the B200 backend
    m.attr("has_vulkan") = true;
    m.attr("device_backend") = "b200";  // lets a caller tell this build from a Vulkan one
    m.def("vulkan_available", [] { return cuda_device_count() > 0; });
    m.def("vulkan_device_count", &cuda_device_count);
    m.def("vulkan_unavailable_reason", &unavailable_reason);
    m.def("vulkan_device_names", [] {
        std::vector<std::string> names;
        for (const b200_caps& c : device_caps()) names.emplace_back(c.name);
        return names;
    });
    m.def("vulkan_device_reports", [] {
        py::list out;
        for (const b200_caps& c : device_caps()) {
            py::dict d;
            const bool usable = c.cc_major == 10;
            d["name"] = std::string(c.name);
            d["driver_name"] = "CUDA (vkml_b200)";
            d["device_type"] = "discrete";
            d["api_version"] = "sm_" + std::to_string(c.cc_major) + std::to_string(c.cc_minor);
            d["driver_version"] = std::to_string(B200_ABI_VERSION);
            d["vendor_id"] = 0x10DE;
            d["device_id"] = 0;
            d["supported"] = usable;
            d["missing_requirement"] = usable ? std::string() : std::string("compute capability 10.x (sm_100a)");
            for (const char* feature : {"buffer_device_address", "scalar_block_layout", "timeline_semaphore",
                                        "synchronization2", "subgroup_size_control", "shader_float16", "shader_int8",
                                        "shader_int16", "storage_buffer_16bit", "global_float_atomic_add",
                                        "shared_float_atomic_add", "cooperative_matrix"}) {
                d[feature] = true;
            }
            d["subgroup_size"] = c.warp_size;
            d["min_subgroup_size"] = c.warp_size;
            d["max_subgroup_size"] = c.warp_size;
            d["max_workgroup_invocations"] = c.max_threads_per_block;
            d["max_workgroup_count_x"] = 2147483647u;
            d["shader_core_count"] = c.sm_count;
            d["max_shared_memory"] = c.max_shared_memory_bytes;
            d["max_push_constants"] = 4096;
            d["max_allocation_size"] = c.total_memory_bytes;
            d["device_local_bytes"] = c.total_memory_bytes;
            d["host_visible_device_local_bytes"] = 0;
            d["timestamp_period"] = 1.0;
            out.append(d);
        }
        return out;
    });
    m.def("init_vulkan", [](int index) { return std::string(device_backend(index).name()); }, "index"_a = 0);
    m.def(
        "vulkan_stats",
        [](int index) {
            b200_stats s{};
            b200_get_stats(device_backend(index).context(), &s);
            py::dict d;
            d["reserved_bytes"] = s.reserved_bytes;
            d["in_use_bytes"] = s.in_use_bytes;
            d["peak_in_use_bytes"] = s.peak_in_use_bytes;
            d["block_count"] = s.driver_allocations;
            d["live_allocations"] = s.live_allocations;
            d["total_allocations"] = s.total_allocations;
            d["device_allocations"] = s.driver_allocations;
            d["fragmentation"] = s.reserved_bytes ? 1.0 - double(s.in_use_bytes) / double(s.reserved_bytes) : 0.0;
            d["submissions"] = s.compute_calls;
            d["dispatches"] = s.kernel_launches;
            d["pipelines"] = 0;
            d["gpu_ms"] = 0.0;
            d["nodes_computed"] = s.nodes_computed;
            d["comm_bytes"] = s.comm_bytes;
            return d;
        },
        "index"_a = 0);
    m.def(
        "vulkan_capabilities",
        [](int index) {
            const vkml::DeviceCapabilities& c = device_backend(index).capabilities();
            return py::dict("fp16_compute"_a = c.fp16_compute, "subgroup_size"_a = c.subgroup_size,
                            "can_pin_subgroup_size"_a = c.can_pin_subgroup_size,
                            "min_subgroup_size"_a = c.min_subgroup_size, "max_subgroup_size"_a = c.max_subgroup_size,
                            "global_float_atomics"_a = c.global_float_atomics,
                            "shared_float_atomics"_a = c.shared_float_atomics,
                            "cooperative_matrix"_a = c.cooperative_matrix,
                            "max_workgroup_invocations"_a = c.max_workgroup_invocations,
                            "max_shared_memory_bytes"_a = c.max_shared_memory_bytes,
                            "total_memory_bytes"_a = c.total_memory_bytes);
        },
        "index"_a = 0);
    m.def("vulkan_timestamps_supported", [](int) { return true; }, "index"_a = 0);
    m.def(
        "vulkan_set_profiling",
        [](bool on, int index) { b200_profile_enable(device_backend(index).context(), on ? 1 : 0); }, "enabled"_a,
        "index"_a = 0);
    m.def(
        "vulkan_last_profile",
        [](int index) {
            std::vector<std::pair<std::string, double>> out;
            for (const ProfileRecord& r : read_profile(index).last) out.emplace_back(r.label, r.gpu_ms);
            return out;
        },
        "index"_a = 0);
    m.def(
        "vulkan_profile_records",
        [](int index) {
            py::list out;
            for (const ProfileRecord& r : read_profile(index).last) out.append(record_dict(r));
            return out;
        },
        "index"_a = 0);
    m.def(
        "vulkan_set_profile_history",
        [](size_t submissions, int index) {
            ProfileStore& store = read_profile(index);  // what ran so far belongs to the old window
            store.keep = submissions;
            store.history.clear();
            store.resolved = 0;
        },
        "submissions"_a, "index"_a = 0);
    m.def(
        "vulkan_profile_history",
        [](int index) {
            py::list out;
            for (const auto& group : read_profile(index).history) {
                for (const ProfileRecord& r : group) out.append(record_dict(r));
            }
            return out;
        },
        "index"_a = 0);
    m.def("vulkan_profile_submissions_resolved", [](int index) { return read_profile(index).resolved; }, "index"_a = 0);
    m.def("vulkan_synchronize", [](int index) { device_backend(index).synchronize(); }, "index"_a = 0);
    // A warp is 32 lanes and cannot be resized; accepted so callers written for vkML's device run.
    m.def("vulkan_set_subgroup_override", [](uint32_t, int) {}, "size"_a, "index"_a = 0);
    m.def("vulkan_pipeline_stats", [](int) { return py::list(); }, "index"_a = 0);

    // -- B200 extras (no counterpart in vkML)
    m.def(
        "b200_set_gemm_precision",
        [](const std::string& precision, int index) {
            const int code = precision == "3xtf32" ? B200_GEMM_3XTF32 : precision == "tf32" ? B200_GEMM_TF32
                             : precision == "fp32" ? B200_GEMM_FP32 : -1;
            if (code < 0) throw vkml::Error("precision must be 3xtf32, tf32 or fp32");
            b200_set_gemm_precision(device_backend(index).context(), code);
        },
        "precision"_a, "index"_a = 0);
    m.def("b200_arm_grad_sync", [](int index) { device_backend(index).arm_grad_sync(); }, "index"_a = 0);
}
