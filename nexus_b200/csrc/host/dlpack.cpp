// DLPack v0.8 producer and consumer, written against the public struct layout (dmlc/dlpack, dlpack.h).
// Export wraps a raw buffer (pointer, shape, strides in elements, device) in a "dltensor" capsule and keeps a Python
// owner object alive until the consumer runs the deleter.  Import validates a capsule (F32, one lane, CPU / CUDA /
// CUDA-host device, non-negative extents), renames it "used_dltensor" as the protocol demands and hands back the
// geometry plus a keeper whose destruction runs the producer's deleter.
// Parity: include/nexus/interop/dlpack.hpp of the reference (v0.8 layout, F32 only, zero copy).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstdint>
#include <memory>
#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

extern "C" {
struct DlDevice { int32_t device_type; int32_t device_id; };
struct DlDataType { uint8_t code; uint8_t bits; uint16_t lanes; };
struct DlTensor {
  void* data;
  DlDevice device;
  int32_t ndim;
  DlDataType dtype;
  int64_t* shape;
  int64_t* strides;
  uint64_t byte_offset;
};
struct DlManagedTensor {
  DlTensor dl_tensor;
  void* manager_ctx;
  void (*deleter)(DlManagedTensor*);
};
}

constexpr int kCpu = 1, kCuda = 2, kCudaHost = 3;
constexpr uint8_t kFloat = 2;
constexpr const char* kFresh = "dltensor";
constexpr const char* kUsed = "used_dltensor";

struct ExportCtx {
  DlManagedTensor managed{};
  std::vector<int64_t> shape, strides;
  PyObject* owner = nullptr;
};

void export_deleter(DlManagedTensor* m) {
  auto* ctx = static_cast<ExportCtx*>(m->manager_ctx);
  if (ctx->owner != nullptr && Py_IsInitialized()) {
    py::gil_scoped_acquire gil;     // a consumer may drop its last reference on any thread
    Py_DECREF(ctx->owner);
  }
  delete ctx;
}

void capsule_destructor(PyObject* cap) {
  // a capsule nobody consumed still owns the tensor; a consumed one was renamed and owns nothing
  if (!PyCapsule_IsValid(cap, kFresh)) return;
  auto* m = static_cast<DlManagedTensor*>(PyCapsule_GetPointer(cap, kFresh));
  if (m != nullptr && m->deleter != nullptr) m->deleter(m);
}

py::object dlpack_export(uintptr_t ptr, const std::vector<int64_t>& shape, const std::vector<int64_t>& strides, int bits,
                         int device_type, int device_id, py::object owner) {
  if (bits != 32) throw std::invalid_argument("dlpack: export supports FP32 tensors");
  if (device_type != kCpu && device_type != kCuda && device_type != kCudaHost)
    throw std::invalid_argument("dlpack: device must be CPU, CUDA or CUDA host");
  if (!strides.empty() && strides.size() != shape.size()) throw std::invalid_argument("dlpack: strides do not match the shape");
  int64_t numel = 1;
  for (int64_t d : shape) {
    if (d < 0) throw std::invalid_argument("dlpack: negative extent");
    numel *= d;
  }
  if (ptr == 0 && numel != 0) throw std::invalid_argument("dlpack: null data pointer");
  auto ctx = std::make_unique<ExportCtx>();
  ctx->shape = shape;
  ctx->strides = strides;
  DlTensor& t = ctx->managed.dl_tensor;
  t.data = reinterpret_cast<void*>(ptr);
  t.device = {device_type, device_id};
  t.ndim = static_cast<int32_t>(shape.size());
  t.dtype = {kFloat, 32, 1};
  t.shape = ctx->shape.data();
  t.strides = strides.empty() ? nullptr : ctx->strides.data();
  t.byte_offset = 0;
  ctx->managed.manager_ctx = ctx.get();
  ctx->managed.deleter = &export_deleter;
  PyObject* cap = PyCapsule_New(&ctx->managed, kFresh, &capsule_destructor);
  if (cap == nullptr) throw py::error_already_set();
  ctx->owner = owner.release().ptr();      // reference handed to the capsule
  ctx.release();
  return py::reinterpret_steal<py::object>(cap);
}

// Runs the producer's deleter once, when the last user of the imported memory lets go.
struct Keeper {
  DlManagedTensor* managed = nullptr;
  ~Keeper() { release(); }
  void release() {
    if (managed != nullptr && managed->deleter != nullptr) managed->deleter(managed);
    managed = nullptr;
  }
};

py::dict dlpack_import(py::object capsule) {
  PyObject* cap = capsule.ptr();
  if (!PyCapsule_CheckExact(cap)) throw std::invalid_argument("dlpack: expected a capsule");
  if (!PyCapsule_IsValid(cap, kFresh)) {
    const char* name = PyCapsule_GetName(cap);
    if (name != nullptr && std::string(name) == kUsed) throw std::invalid_argument("dlpack: capsule was already consumed");
    throw std::invalid_argument("dlpack: capsule is not a dltensor");
  }
  auto* m = static_cast<DlManagedTensor*>(PyCapsule_GetPointer(cap, kFresh));
  if (m == nullptr) throw py::error_already_set();
  const DlTensor& t = m->dl_tensor;
  // validation first: a refused capsule stays unconsumed and with its producer
  if (t.dtype.code != kFloat || t.dtype.bits != 32 || t.dtype.lanes != 1) throw std::invalid_argument("dlpack: import supports FP32 tensors");
  if (t.device.device_type != kCpu && t.device.device_type != kCuda && t.device.device_type != kCudaHost)
    throw std::invalid_argument("dlpack: unsupported device type " + std::to_string(t.device.device_type));
  if (t.ndim < 0 || (t.ndim > 0 && t.shape == nullptr)) throw std::invalid_argument("dlpack: bad shape");
  std::vector<int64_t> shape(t.shape, t.shape + t.ndim), strides(static_cast<size_t>(t.ndim));
  int64_t numel = 1;
  for (int64_t d : shape) {
    if (d < 0) throw std::invalid_argument("dlpack: negative extent");
    numel *= d;
  }
  if (t.strides != nullptr) {
    for (int i = 0; i < t.ndim; ++i) {
      if (t.strides[i] < 0) throw std::invalid_argument("dlpack: negative strides are not supported");
      strides[static_cast<size_t>(i)] = t.strides[i];
    }
  } else {
    int64_t s = 1;
    for (int i = t.ndim - 1; i >= 0; --i) {
      strides[static_cast<size_t>(i)] = s;
      s *= shape[static_cast<size_t>(i)];
    }
  }
  if (t.data == nullptr && numel != 0) throw std::invalid_argument("dlpack: null data pointer");
  if (t.byte_offset % 4 != 0) throw std::invalid_argument("dlpack: byte offset is not a multiple of the element size");
  int64_t span = numel == 0 ? 0 : 1;       // elements from the first to one past the last addressed
  for (int i = 0; i < t.ndim && numel != 0; ++i) span += (shape[static_cast<size_t>(i)] - 1) * strides[static_cast<size_t>(i)];
  if (PyCapsule_SetName(cap, kUsed) != 0) throw py::error_already_set();
  auto keeper = std::make_shared<Keeper>();
  keeper->managed = m;
  py::dict out;
  out["ptr"] = reinterpret_cast<uintptr_t>(t.data) + t.byte_offset;
  out["shape"] = shape;
  out["strides"] = strides;
  out["span"] = span;
  out["device_type"] = t.device.device_type;
  out["device_id"] = t.device.device_id;
  out["keeper"] = py::cast(keeper);
  return out;
}

}  // namespace

void bind_dlpack(py::module_& m) {
  py::class_<Keeper, std::shared_ptr<Keeper>>(m, "DlpackKeeper")
      .def("release", &Keeper::release)
      .def_property_readonly("alive", [](const Keeper& k) { return k.managed != nullptr; });
  m.def("dlpack_export", &dlpack_export, py::arg("ptr"), py::arg("shape"), py::arg("strides"), py::arg("bits"),
        py::arg("device_type"), py::arg("device_id"), py::arg("owner"));
  m.def("dlpack_import", &dlpack_import);
}
