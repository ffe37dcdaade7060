// _infinicore_b200: the Python module over the C++ host layer (include/infinicore_b200/ops.hpp), with the
// operator signatures of the reference's pybind layer for this path
// (src/infinicore/pybind11/ops/paged_attention.hpp:11-55, src/infinicore/pybind11/ops/paged_caching.hpp:11-22):
//     paged_attention(q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes, scale) -> Tensor
//     paged_attention_(out, q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes, scale)
//     paged_caching_(k_cache, v_cache, k, v, slot_mapping)
// and, beside them, the prefill operator, the status word and the stream the calls run on.
//
// A Tensor here is what the operators need and nothing more: a device pointer with dtype, shape and element
// strides - either a view of memory somebody else owns (from_blob: a torch tensor, a framework buffer) or memory
// obtained from infinirtMalloc (empty), released when the last Python reference goes.  The reference's Tensor
// class with its allocator, views and printing is not rebuilt.
//
// Plain C++17 (no CUDA headers): compiled with g++ against pybind11, linked to libinfiniop / libinfinirt.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "infinicore_b200/ops.hpp"

#include <memory>
#include <optional>
#include <sstream>
#include <string>
#include <vector>

namespace py = pybind11;
namespace ib = infinicore_b200;

namespace {

// the stream every call of the calling thread goes to (NULL: the default stream), as the reference's
// context keeps a current stream per thread (include/infinicore/context/context.hpp)
thread_local infinirtStream_t t_stream = nullptr;

size_t elementSize(infiniDtype_t dt) {
    switch (dt) {
    case INFINI_DTYPE_BYTE:
    case INFINI_DTYPE_BOOL:
    case INFINI_DTYPE_I8:
    case INFINI_DTYPE_U8:
    case INFINI_DTYPE_F8:
        return 1;
    case INFINI_DTYPE_I16:
    case INFINI_DTYPE_U16:
    case INFINI_DTYPE_F16:
    case INFINI_DTYPE_BF16:
        return 2;
    case INFINI_DTYPE_I32:
    case INFINI_DTYPE_U32:
    case INFINI_DTYPE_F32:
        return 4;
    case INFINI_DTYPE_I64:
    case INFINI_DTYPE_U64:
    case INFINI_DTYPE_F64:
        return 8;
    default:
        return 0;
    }
}

class PyTensor {
public:
    PyTensor(ib::Tensor view, int device_index, std::shared_ptr<void> owner)
        : view_(std::move(view)), device_index_(device_index), owner_(std::move(owner)) {}

    static PyTensor fromBlob(uintptr_t data, std::vector<size_t> shape, std::optional<std::vector<ptrdiff_t>> strides,
                             infiniDtype_t dtype, int device_index) {
        if (elementSize(dtype) == 0) {
            throw std::invalid_argument("from_blob: unknown dtype");
        }
        if (strides.has_value() && strides->size() != shape.size()) {
            throw std::invalid_argument("from_blob: strides and shape differ in length");
        }
        void *ptr = reinterpret_cast<void *>(data);
        ib::Tensor t = strides.has_value() ? ib::Tensor(ptr, dtype, std::move(shape), std::move(*strides)) : ib::Tensor(ptr, dtype, std::move(shape));
        return PyTensor(std::move(t), device_index, nullptr);
    }

    static PyTensor empty(std::vector<size_t> shape, infiniDtype_t dtype, int device_index) {
        const size_t es = elementSize(dtype);
        if (es == 0) {
            throw std::invalid_argument("empty: unknown dtype");
        }
        size_t n = 1;
        for (size_t d : shape) {
            n *= d;
        }
        ib::check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, device_index), "infinirtSetDevice");
        void *ptr = nullptr;
        if (n > 0) {
            ib::check(infinirtMalloc(&ptr, n * es), "infinirtMalloc");
        }
        std::shared_ptr<void> owner(ptr, [](void *p) {
            if (p != nullptr) {
                infinirtFree(p);
            }
        });
        return PyTensor(ib::Tensor(ptr, dtype, std::move(shape)), device_index, std::move(owner));
    }

    const ib::Tensor &view() const { return view_; }
    int deviceIndex() const { return device_index_; }
    uintptr_t dataPtr() const { return reinterpret_cast<uintptr_t>(view_.data); }
    size_t numel() const {
        size_t n = 1;
        for (size_t d : view_.shape) {
            n *= d;
        }
        return n;
    }
    std::string repr() const {
        std::ostringstream os;
        os << "Tensor(shape=[";
        for (size_t i = 0; i < view_.shape.size(); ++i) {
            os << (i ? ", " : "") << view_.shape[i];
        }
        os << "], strides=[";
        for (size_t i = 0; i < view_.strides.size(); ++i) {
            os << (i ? ", " : "") << view_.strides[i];
        }
        os << "], dtype=" << static_cast<int>(view_.dtype) << ", device=nvidia:" << device_index_ << (owner_ ? ", owning" : ", view") << ")";
        return os.str();
    }

private:
    ib::Tensor view_;
    int device_index_;
    std::shared_ptr<void> owner_;
};

// All tensors of a call live on one device; the calling thread's infinirt device follows them.
void enterDevice(std::initializer_list<const PyTensor *> tensors) {
    int device = -1;
    for (const PyTensor *t : tensors) {
        if (t == nullptr) {
            continue;
        }
        if (device < 0) {
            device = t->deviceIndex();
        } else if (t->deviceIndex() != device) {
            throw std::invalid_argument("all tensors of one call must live on the same device");
        }
    }
    ib::check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, device < 0 ? 0 : device), "infinirtSetDevice");
}

std::optional<ib::Tensor> optionalView(const py::object &o, const PyTensor **keep) {
    *keep = nullptr;
    if (o.is_none()) {
        return std::nullopt;
    }
    const PyTensor &t = o.cast<const PyTensor &>();
    *keep = &t;
    return t.view();
}

void pagedAttentionInto(const PyTensor &out, const PyTensor &q, const PyTensor &k_cache, const PyTensor &v_cache,
                        const PyTensor &block_tables, const PyTensor &cache_lens, const py::object &alibi_slopes, float scale) {
    const PyTensor *alibi = nullptr;
    std::optional<ib::Tensor> slopes = optionalView(alibi_slopes, &alibi);
    enterDevice({&out, &q, &k_cache, &v_cache, &block_tables, &cache_lens, alibi});
    py::gil_scoped_release release;
    ib::op::paged_attention_(out.view(), q.view(), k_cache.view(), v_cache.view(), block_tables.view(), cache_lens.view(), slopes, scale, t_stream);
}

PyTensor pagedAttention(const PyTensor &q, const PyTensor &k_cache, const PyTensor &v_cache, const PyTensor &block_tables,
                        const PyTensor &cache_lens, const py::object &alibi_slopes, float scale) {
    if (q.view().shape.size() != 3 || v_cache.view().shape.size() != 4) {
        throw std::invalid_argument("paged_attention: q must be [seqs, heads, head], v_cache [blocks, kv_heads, block, value]");
    }
    // out takes the value width, as the reference's wrapper does (src/infinicore/ops/paged_attention/paged_attention.cc)
    PyTensor out = PyTensor::empty({q.view().shape[0], q.view().shape[1], v_cache.view().shape[3]}, q.view().dtype, q.deviceIndex());
    pagedAttentionInto(out, q, k_cache, v_cache, block_tables, cache_lens, alibi_slopes, scale);
    return out;
}

void pagedCachingInto(const PyTensor &k_cache, const PyTensor &v_cache, const PyTensor &k, const PyTensor &v, const PyTensor &slot_mapping) {
    enterDevice({&k_cache, &v_cache, &k, &v, &slot_mapping});
    py::gil_scoped_release release;
    ib::op::paged_caching_(k_cache.view(), v_cache.view(), k.view(), v.view(), slot_mapping.view(), t_stream);
}

void pagedAttentionPrefillInto(const PyTensor &out, const PyTensor &q, const PyTensor &k_cache, const PyTensor &v_cache,
                               const PyTensor &block_tables, const PyTensor &total_kv_lens, const PyTensor &cum_seqlens_q,
                               const py::object &alibi_slopes, float scale) {
    const PyTensor *alibi = nullptr;
    std::optional<ib::Tensor> slopes = optionalView(alibi_slopes, &alibi);
    enterDevice({&out, &q, &k_cache, &v_cache, &block_tables, &total_kv_lens, &cum_seqlens_q, alibi});
    py::gil_scoped_release release;
    ib::op::paged_attention_prefill_(out.view(), q.view(), k_cache.view(), v_cache.view(), block_tables.view(), total_kv_lens.view(),
                                     cum_seqlens_q.view(), slopes, scale, t_stream);
}

} // namespace

PYBIND11_MODULE(_infinicore_b200, m) {
    m.doc() = "Paged decode path of InfiniCore on B200: paged_attention / paged_caching_ over libinfiniop (no CPU path)";

    py::register_exception<ib::StatusError>(m, "StatusError", PyExc_RuntimeError);

    py::enum_<infiniDtype_t>(m, "DataType")
        .value("BOOL", INFINI_DTYPE_BOOL)
        .value("I8", INFINI_DTYPE_I8)
        .value("I16", INFINI_DTYPE_I16)
        .value("I32", INFINI_DTYPE_I32)
        .value("I64", INFINI_DTYPE_I64)
        .value("U8", INFINI_DTYPE_U8)
        .value("U32", INFINI_DTYPE_U32)
        .value("U64", INFINI_DTYPE_U64)
        .value("F16", INFINI_DTYPE_F16)
        .value("F32", INFINI_DTYPE_F32)
        .value("F64", INFINI_DTYPE_F64)
        .value("BF16", INFINI_DTYPE_BF16);

    py::class_<PyTensor>(m, "Tensor")
        .def_static("from_blob", &PyTensor::fromBlob, py::arg("data_ptr"), py::arg("shape"), py::arg("strides") = py::none(), py::arg("dtype"),
                    py::arg("device_index") = 0,
                    "A view of device memory the caller owns and keeps alive; strides in elements (None: contiguous).")
        .def_static("empty", &PyTensor::empty, py::arg("shape"), py::arg("dtype"), py::arg("device_index") = 0,
                    "Contiguous device memory from infinirtMalloc, freed with the last reference.")
        .def("data_ptr", &PyTensor::dataPtr)
        .def("numel", &PyTensor::numel)
        .def_property_readonly("shape", [](const PyTensor &t) { return t.view().shape; })
        .def_property_readonly("strides", [](const PyTensor &t) { return t.view().strides; })
        .def_property_readonly("dtype", [](const PyTensor &t) { return t.view().dtype; })
        .def_property_readonly("device_index", &PyTensor::deviceIndex)
        .def("__repr__", &PyTensor::repr);

    m.def("paged_attention", &pagedAttention, py::arg("q"), py::arg("k_cache"), py::arg("v_cache"), py::arg("block_tables"),
          py::arg("cache_lens"), py::arg("alibi_slopes"), py::arg("scale"), R"doc(Paged attention of query and key cache tensors.)doc");
    m.def("paged_attention_", &pagedAttentionInto, py::arg("out"), py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("block_tables"), py::arg("cache_lens"), py::arg("alibi_slopes"), py::arg("scale"),
          R"doc(In-place paged attention of query and key cache tensors.)doc");
    m.def("paged_caching_", &pagedCachingInto, py::arg("k_cache"), py::arg("v_cache"), py::arg("k"), py::arg("v"), py::arg("slot_mapping"),
          R"doc(Paged caching of key and value tensors.)doc");
    m.def("paged_attention_prefill_", &pagedAttentionPrefillInto, py::arg("out"), py::arg("q"), py::arg("k_cache"), py::arg("v_cache"),
          py::arg("block_tables"), py::arg("total_kv_lens"), py::arg("cum_seqlens_q"), py::arg("alibi_slopes"), py::arg("scale"),
          R"doc(In-place causal attention of packed new tokens over the paged cache that already holds them.)doc");

    m.def("set_stream", [](uintptr_t stream) { t_stream = reinterpret_cast<infinirtStream_t>(stream); }, py::arg("stream"),
          "The stream (a cudaStream_t as an integer; 0: the default stream) the calling thread's calls go to.");
    m.def("get_stream", []() { return reinterpret_cast<uintptr_t>(t_stream); });
    m.def("sync_stream", []() {
        py::gil_scoped_release release;
        ib::check(infinirtStreamSynchronize(t_stream), "infinirtStreamSynchronize");
    });
    m.def("sync_device", []() {
        py::gil_scoped_release release;
        ib::check(infinirtDeviceSynchronize(), "infinirtDeviceSynchronize");
    });
    m.def("set_device", [](int index) { ib::check(infinirtSetDevice(INFINI_DEVICE_NVIDIA, index), "infinirtSetDevice"); }, py::arg("index"));
    m.def("kernel_status", []() { return ib::kernel_status(t_stream); },
          "Waits for the calling thread's stream, returns the device's kernel status flags and clears them (0: all work done).");
    m.def("cached_descriptors", []() { return ib::cached_descriptors(); });
    m.def("clear_cache", []() { ib::clear_cache(); });
}
