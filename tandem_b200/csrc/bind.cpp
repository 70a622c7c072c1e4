// Python bindings of the host runtime (module tandem_b200._host).
//
// The Python-visible surface is the one the reference's module exposes (tandem/csrc/engine.cpp:53-123:
// SharedMemory, Channel, Work, Engine, _move_check, the Timeout / NotImplemented mappings), because the
// package's Python layer and its tests are written against it.  Tensors cross as (address, element count,
// dtype code), so this module does not link against libtorch; every call that can wait releases the GIL.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <string_view>
#include <type_traits>

#include "channel.h"
#include "engine.h"
#include "shm.h"

namespace py = pybind11;

namespace {

using tb::Channel;
using tb::DType;
using tb::Engine;
using tb::SharedMemory;
using tb::Work;

// One owner per mapping, and handing it over cannot fail: checked where the bindings are compiled.
static_assert(!std::is_copy_constructible_v<SharedMemory> && !std::is_copy_assignable_v<SharedMemory>, "a mapping has one owner");
static_assert(std::is_nothrow_move_constructible_v<SharedMemory> && std::is_nothrow_move_assignable_v<SharedMemory>,
              "moving a mapping cannot fail");

inline void* at_address(std::uintptr_t address) { return reinterpret_cast<void*>(address); }

// The bytes [offset, offset + count) of a live region, or an exception saying why not.
char* span_of(const SharedMemory& region, std::size_t offset, std::size_t count) {
  if (region.data() == nullptr) throw std::invalid_argument("the region is closed");
  if (offset > region.size() || count > region.size() - offset) throw std::out_of_range("outside the region");
  return static_cast<char*>(region.data()) + offset;
}

// Move construction and move assignment cannot be reached from Python; this walks a mapping through both and
// reports what it saw.  (Keys as in the reference's _move_check, which the shared-memory tests read.)
py::dict move_check(const std::string& first_name, const std::string& second_name) {
  constexpr std::size_t kBytes = 4096;
  py::dict seen;
  SharedMemory origin = SharedMemory::create(first_name, kBytes);
  void* const mapping = origin.data();

  SharedMemory heir(std::move(origin));
  seen["source_emptied"] = origin.data() == nullptr && origin.size() == 0 && !origin.owner();
  seen["target_took_over"] = heir.data() == mapping && heir.size() == kBytes && heir.owner();

  SharedMemory other = SharedMemory::create(second_name, kBytes);
  other = std::move(heir);  // lets go of second_name's region, then holds first_name's
  seen["assigned"] = other.data() == mapping && other.name() == first_name && heir.data() == nullptr;

  SharedMemory& itself = other;
  other = std::move(itself);
  seen["self_assign_safe"] = other.data() == mapping;
  return seen;
}

void bind_shared_memory(py::module_& m) {
  py::class_<SharedMemory> cls(m, "SharedMemory");
  cls.def_static("create", &SharedMemory::create, py::arg("name"), py::arg("bytes"));
  cls.def_static("open", &SharedMemory::open, py::arg("name"));
  cls.def("close", &SharedMemory::drop);
  cls.def_property_readonly("name", &SharedMemory::name);
  cls.def_property_readonly("size", &SharedMemory::size);
  cls.def_property_readonly("owner", &SharedMemory::owner);
  cls.def_property_readonly("closed", [](const SharedMemory& region) { return region.data() == nullptr; });
  cls.def_property_readonly("address", [](const SharedMemory& region) { return reinterpret_cast<std::uintptr_t>(region.data()); });
  cls.def("read", [](const SharedMemory& region, std::size_t offset, std::size_t count) {
    return py::bytes(span_of(region, offset, count), count);
  });
  cls.def("write", [](SharedMemory& region, std::size_t offset, const py::bytes& payload) {
    const std::string_view bytes = payload;
    char* target = span_of(region, offset, bytes.size());
    if (!bytes.empty()) std::memcpy(target, bytes.data(), bytes.size());
  });
}

void bind_channel(py::module_& m) {
  py::class_<Channel> cls(m, "Channel");
  cls.def_static("create", &Channel::create, py::arg("name"), py::arg("slots"), py::arg("slot_bytes"));
  cls.def_static("open", &Channel::open, py::arg("name"));
  cls.def_property_readonly("slots", &Channel::slot_count);
  cls.def_property_readonly("slot_bytes", &Channel::slot_capacity);
  cls.def(
      "send",
      [](Channel& channel, const py::bytes& payload, double timeout) {
        const std::string message = payload;  // copied out while the GIL is still held
        py::gil_scoped_release unlocked;
        channel.send(message.data(), message.size(), timeout);
      },
      py::arg("data"), py::arg("timeout") = 10.0);
  cls.def(
      "recv",
      [](Channel& channel, std::size_t capacity, double timeout) {
        std::string room(capacity, '\0');
        std::size_t got = 0;
        {
          py::gil_scoped_release unlocked;
          got = channel.recv(room.data(), capacity, timeout);
        }
        return py::bytes(room.data(), got);
      },
      py::arg("capacity"), py::arg("timeout") = 10.0);
}

void bind_work(py::module_& m) {
  py::class_<Work, std::shared_ptr<Work>> cls(m, "Work");
  cls.def("wait", &Work::wait, py::call_guard<py::gil_scoped_release>());
  cls.def("done", &Work::done);
  cls.def_property_readonly("started", &Work::started);
  cls.def_property_readonly("finished", &Work::finished);
}

// A Python callable queued on the progress thread.  The thread takes the GIL to call it and to let go of it.
class PythonJob {
 public:
  explicit PythonJob(py::function fn) : fn_(std::move(fn)) {}
  PythonJob(const PythonJob&) = delete;
  PythonJob& operator=(const PythonJob&) = delete;
  ~PythonJob() {
    py::gil_scoped_acquire locked;
    fn_ = py::function();
  }
  void run() {
    py::gil_scoped_acquire locked;
    fn_();
  }

 private:
  py::function fn_;
};

void bind_engine(py::module_& m) {
  using Address = std::uintptr_t;
  using Count = std::int64_t;
  py::class_<Engine> cls(m, "Engine");
  cls.def(py::init<const std::string&, int, int, std::size_t, std::size_t, double>(), py::arg("job"), py::arg("rank"), py::arg("size"),
          py::arg("slots"), py::arg("slot_bytes"), py::arg("timeout"));
  cls.def_property_readonly("rank", &Engine::rank);
  cls.def_property_readonly("size", &Engine::size);
  cls.def("connect", &Engine::connect, py::call_guard<py::gil_scoped_release>());
  cls.def("close", &Engine::close, py::call_guard<py::gil_scoped_release>());
  cls.def("abort", &Engine::abort);
  cls.def("barrier", &Engine::barrier);
  // collectives over `numel` elements of dtype code `dtype` at `data`
  cls.def("all_reduce", [](Engine& engine, Address data, Count numel, int dtype, bool average) {
    return engine.all_reduce(at_address(data), numel, DType(dtype), average);
  });
  cls.def("reduce_scatter", [](Engine& engine, Address data, Count numel, int dtype, Engine::Sizes sizes, bool average) {
    return engine.reduce_scatter(at_address(data), numel, DType(dtype), std::move(sizes), average);
  });
  cls.def("all_gather", [](Engine& engine, Address data, Count numel, int dtype, Engine::Sizes sizes) {
    return engine.all_gather(at_address(data), numel, DType(dtype), std::move(sizes));
  });
  cls.def("broadcast", [](Engine& engine, Address data, Count numel, int dtype, int root) {
    return engine.broadcast(at_address(data), numel, DType(dtype), root);
  });
  // point to point, in bytes
  cls.def("send", [](Engine& engine, Address data, Count nbytes, int to) { return engine.send(at_address(data), nbytes, to); });
  cls.def("recv", [](Engine& engine, Address data, Count nbytes, int from) { return engine.recv(at_address(data), nbytes, from); });
  cls.def("sendrecv", [](Engine& engine, Address out, Count out_bytes, int to, Address in, Count in_bytes, int from) {
    return engine.sendrecv(at_address(out), out_bytes, to, at_address(in), in_bytes, from);
  });
  // an arbitrary Python job, in order with the collectives
  cls.def("submit", [](Engine& engine, py::function fn) {
    auto job = std::make_shared<PythonJob>(std::move(fn));
    return engine.submit([job] { job->run(); });
  });
}

}  // namespace

PYBIND11_MODULE(_host, m) {
  m.doc() = "tandem_b200 host runtime: shared memory, channels, progress thread, CPU collectives";
  py::register_exception<tb::Timeout>(m, "Timeout", PyExc_TimeoutError);
  py::register_exception<tb::Aborted>(m, "Aborted", PyExc_RuntimeError);
  py::register_exception<tb::NotImplemented>(m, "NotImplemented", PyExc_NotImplementedError);
  m.attr("cuda") = false;  // the GPU kernels live in libtb200_cuda.so, loaded separately
  m.def("_move_check", &move_check);
  bind_shared_memory(m);
  bind_channel(m);
  bind_work(m);
  bind_engine(m);
}
