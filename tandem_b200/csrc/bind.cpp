// Python bindings of the host runtime (module tandem_b200._host).
// Surface parity with the reference's tandem/csrc/engine.cpp:53-123; tensors
// cross as (address, element count, dtype code), so this module does not link
// against libtorch.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <cstring>
#include <type_traits>

#include "channel.h"
#include "engine.h"
#include "shm.h"

namespace py = pybind11;
using tb::Channel;
using tb::DType;
using tb::Engine;
using tb::SharedMemory;
using tb::Work;

static_assert(!std::is_copy_constructible_v<SharedMemory> && !std::is_copy_assignable_v<SharedMemory>,
              "a mapping has one owner");
static_assert(std::is_nothrow_move_constructible_v<SharedMemory> && std::is_nothrow_move_assignable_v<SharedMemory>,
              "moving a mapping cannot fail");

namespace {

void in_range(const SharedMemory& s, std::size_t at, std::size_t n) {
  if (s.data() == nullptr) throw std::invalid_argument("the region is closed");
  if (at > s.size() || n > s.size() - at) throw std::out_of_range("outside the region");
}

// Drives the move constructor and move assignment, which Python cannot reach.
py::dict move_check(const std::string& first, const std::string& second) {
  py::dict r;
  SharedMemory a = SharedMemory::create(first, 4096);
  void* where = a.data();
  SharedMemory b(std::move(a));
  r["source_emptied"] = a.data() == nullptr && a.size() == 0 && !a.owner();
  r["target_took_over"] = b.data() == where && b.size() == 4096 && b.owner();
  SharedMemory c = SharedMemory::create(second, 4096);
  c = std::move(b);  // must let go of `second` before taking `first`
  r["assigned"] = c.data() == where && c.name() == first && b.data() == nullptr;
  SharedMemory& same = c;
  c = std::move(same);
  r["self_assign_safe"] = c.data() == where;
  return r;
}

void* ptr(std::uintptr_t address) { return reinterpret_cast<void*>(address); }

}  // namespace

PYBIND11_MODULE(_host, m) {
  m.doc() = "tandem_b200 host runtime: shared memory, channels, progress thread, CPU collectives";
  py::register_exception<tb::NotImplemented>(m, "NotImplemented", PyExc_NotImplementedError);
  py::register_exception<tb::Timeout>(m, "Timeout", PyExc_TimeoutError);
  py::register_exception<tb::Aborted>(m, "Aborted", PyExc_RuntimeError);

  py::class_<SharedMemory>(m, "SharedMemory")
      .def_static("create", &SharedMemory::create, py::arg("name"), py::arg("bytes"))
      .def_static("open", &SharedMemory::open, py::arg("name"))
      .def_property_readonly("size", &SharedMemory::size)
      .def_property_readonly("name", &SharedMemory::name)
      .def_property_readonly("owner", &SharedMemory::owner)
      .def_property_readonly("closed", [](const SharedMemory& s) { return s.data() == nullptr; })
      .def_property_readonly("address", [](const SharedMemory& s) { return reinterpret_cast<std::uintptr_t>(s.data()); })
      .def("write",
           [](SharedMemory& s, std::size_t at, const py::bytes& b) {
             std::string v = b;
             in_range(s, at, v.size());
             std::memcpy(static_cast<char*>(s.data()) + at, v.data(), v.size());
           })
      .def("read",
           [](const SharedMemory& s, std::size_t at, std::size_t n) {
             in_range(s, at, n);
             return py::bytes(static_cast<const char*>(s.data()) + at, n);
           })
      .def("close", &SharedMemory::drop);

  m.def("_move_check", &move_check);
  m.attr("cuda") = false;  // GPU kernels live in libtb200_cuda.so, loaded separately

  py::class_<Channel>(m, "Channel")
      .def_static("create", &Channel::create, py::arg("name"), py::arg("slots"), py::arg("slot_bytes"))
      .def_static("open", &Channel::open, py::arg("name"))
      .def_property_readonly("slots", &Channel::slot_count)
      .def_property_readonly("slot_bytes", &Channel::slot_capacity)
      .def(
          "send",
          [](Channel& c, const py::bytes& b, double timeout) {
            std::string v = b;
            py::gil_scoped_release unlocked;
            c.send(v.data(), v.size(), timeout);
          },
          py::arg("data"), py::arg("timeout") = 10.0)
      .def(
          "recv",
          [](Channel& c, std::size_t capacity, double timeout) {
            std::string buf(capacity, '\0');
            std::size_t n;
            {
              py::gil_scoped_release unlocked;
              n = c.recv(buf.data(), capacity, timeout);
            }
            return py::bytes(buf.data(), n);
          },
          py::arg("capacity"), py::arg("timeout") = 10.0);

  py::class_<Work, std::shared_ptr<Work>>(m, "Work")
      .def("wait", &Work::wait, py::call_guard<py::gil_scoped_release>())
      .def("done", &Work::done)
      .def_property_readonly("started", &Work::started)
      .def_property_readonly("finished", &Work::finished);

  py::class_<Engine>(m, "Engine")
      .def(py::init<const std::string&, int, int, std::size_t, std::size_t, double>(), py::arg("job"), py::arg("rank"),
           py::arg("size"), py::arg("slots"), py::arg("slot_bytes"), py::arg("timeout"))
      .def("connect", &Engine::connect, py::call_guard<py::gil_scoped_release>())
      .def("close", &Engine::close, py::call_guard<py::gil_scoped_release>())
      .def("abort", &Engine::abort)
      .def_property_readonly("rank", &Engine::rank)
      .def_property_readonly("size", &Engine::size)
      .def("all_reduce",
           [](Engine& e, std::uintptr_t p, std::int64_t n, int d, bool avg) { return e.all_reduce(ptr(p), n, DType(d), avg); })
      .def("reduce_scatter",
           [](Engine& e, std::uintptr_t p, std::int64_t n, int d, Engine::Sizes sizes, bool avg) {
             return e.reduce_scatter(ptr(p), n, DType(d), std::move(sizes), avg);
           })
      .def("all_gather",
           [](Engine& e, std::uintptr_t p, std::int64_t n, int d, Engine::Sizes sizes) {
             return e.all_gather(ptr(p), n, DType(d), std::move(sizes));
           })
      .def("broadcast",
           [](Engine& e, std::uintptr_t p, std::int64_t n, int d, int root) { return e.broadcast(ptr(p), n, DType(d), root); })
      .def("send", [](Engine& e, std::uintptr_t p, std::int64_t nbytes, int dst) { return e.send(ptr(p), nbytes, dst); })
      .def("recv", [](Engine& e, std::uintptr_t p, std::int64_t nbytes, int src) { return e.recv(ptr(p), nbytes, src); })
      .def("sendrecv",
           [](Engine& e, std::uintptr_t sp, std::int64_t sb, int dst, std::uintptr_t rp, std::int64_t rb, int src) {
             return e.sendrecv(ptr(sp), sb, dst, ptr(rp), rb, src);
           })
      .def("barrier", &Engine::barrier)
      .def("submit", [](Engine& e, py::function fn) {
        // The callable is owned by a holder whose destructor takes the GIL: the
        // progress thread drops it without holding the interpreter lock.
        struct Holder {
          py::function fn;
          ~Holder() {
            py::gil_scoped_acquire locked;
            fn = py::function();
          }
        };
        auto held = std::make_shared<Holder>(Holder{std::move(fn)});
        return e.submit([held] {
          py::gil_scoped_acquire locked;
          held->fn();
        });
      });
}
