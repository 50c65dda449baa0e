// pybind11 module tensorpipe_b200._C: the C++ API for Python.
//
// Counterpart of the reference's "pytensorpipe" (tensorpipe/python/tensorpipe.cc:229-453), with
// two differences: tensors may live on CUDA devices (they are described by address, length,
// device, stream and dtype, which the Python layer extracts from torch tensors — this module does
// not link against torch), and error callbacks DO reach Python (the reference only logs them).
// The GIL is released around every call into the library and re-acquired inside callbacks; the
// Python callables and the buffers they refer to are kept alive until their callback has run.
#include <pybind11/functional.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <tpb/tpb.h>

#include "kernels/push.h"
#include "tools/ring_bench.h"

namespace py = pybind11;
using namespace tpb;

namespace {

// Takes the GIL for a callback. A thread of the library has no Python thread state of its own:
// the one made for its first callback is kept for the thread's later callbacks (one extra count
// on it, never given back) instead of being built and torn down around every callback, which
// costs more than the callback itself. A Python thread that runs a callback (the on-demand loop
// borrows the calling thread) already has its state and is left alone.
class CallbackGil {
 public:
  CallbackGil() : fresh_(threadHasNoState()), gil_() {
    if (fresh_) gil_.inc_ref();
  }

 private:
  static bool threadHasNoState() {
    return py::detail::get_internals().tstate.get() == nullptr && PyGILState_GetThisThreadState() == nullptr;
  }
  bool fresh_;
  py::gil_scoped_acquire gil_;
};

// Holds Python objects and drops them with the GIL held, wherever the last reference dies.
struct PyKeepAlive {
  std::vector<py::object> objects;
  ~PyKeepAlive() {
    if (objects.empty()) return;
    CallbackGil gil;
    objects.clear();
  }
};

std::string errorString(const Error& e) { return e ? e.what() : std::string(); }

struct PyOutMessage {
  Message msg;
  std::shared_ptr<PyKeepAlive> keep = std::make_shared<PyKeepAlive>();
};

struct PyAllocation {
  Allocation alloc;
  std::shared_ptr<PyKeepAlive> keep = std::make_shared<PyKeepAlive>();
};

Buffer makeBuffer(const std::string& deviceType, int deviceIndex, uint64_t ptr, uint64_t stream) {
  if (deviceType == "cpu") return CpuBuffer{reinterpret_cast<void*>(ptr)};
  if (deviceType == "cuda") return CudaBuffer{reinterpret_cast<void*>(ptr), reinterpret_cast<void*>(stream), deviceIndex};
  throw std::runtime_error("unknown device type " + deviceType);
}

// Wraps a Python callable so it can be invoked from any thread, exactly once.
template <typename... Args>
std::function<void(Args...)> wrapCallback(py::function fn, std::shared_ptr<PyKeepAlive> keep) {
  auto holder = std::make_shared<PyKeepAlive>();
  holder->objects.push_back(std::move(fn));
  return [holder, keep](Args... args) {
    CallbackGil gil;
    try {
      py::function f = py::reinterpret_borrow<py::function>(holder->objects[0]);
      f(args...);
    } catch (py::error_already_set& err) {
      // A callback has nowhere to propagate to: report and carry on.
      err.discard_as_unraisable("tensorpipe_b200 callback");
    }
  };
}

py::dict descriptorToDict(const Descriptor& d) {
  py::dict out;
  out["metadata"] = py::bytes(d.metadata);
  py::list payloads, tensors;
  for (const auto& p : d.payloads) {
    py::dict pd;
    pd["length"] = p.length;
    pd["metadata"] = py::bytes(p.metadata);
    payloads.append(pd);
  }
  for (const auto& t : d.tensors) {
    py::dict td;
    td["length"] = t.length;
    td["metadata"] = py::bytes(t.metadata);
    td["source_device"] = t.sourceDevice.toString();
    td["target_device"] = t.targetDevice ? py::cast(t.targetDevice->toString()) : py::none();
    tensors.append(td);
  }
  out["payloads"] = payloads;
  out["tensors"] = tensors;
  return out;
}

Device parseDevice(const std::string& s) {
  auto pos = s.find(':');
  if (pos == std::string::npos) return Device(s, 0);
  return Device(s.substr(0, pos), std::stoi(s.substr(pos + 1)));
}

}  // namespace

PYBIND11_MODULE(_C, m) {
  m.doc() = "tensorpipe_b200 native module";

  py::class_<transport::Context, std::shared_ptr<transport::Context>>(m, "TransportContext")
      .def("is_viable", &transport::Context::isViable)
      .def("domain_descriptor", [](transport::Context& c) { return c.domainDescriptor(); });
  py::class_<channel::Context, std::shared_ptr<channel::Context>>(m, "ChannelContext")
      .def("is_viable", &channel::Context::isViable);

  m.def("create_uv_transport", &transport::uv::create);
  m.def("create_shm_transport", &transport::shm::create);
  m.def("create_ibv_transport", &transport::ibv::create);
  m.def("create_basic_channel", &channel::basic::create);
  m.def("create_xth_channel", &channel::xth::create);
  m.def("create_cma_channel", &channel::cma::create);
  m.def("create_cuda_basic_channel", &channel::cuda_basic::create);
  m.def("create_cuda_gdr_channel", &channel::cuda_gdr::create);
  {
    const channel::cuda_p2p::Options defaults;
    m.def(
        "create_cuda_p2p_channel",
        [](size_t eagerThreshold, size_t inboxBytes, int maxCtas, bool waitWithKernel, bool useBulkCopy,
           size_t sendOrderMinBytes, size_t hostCopyMinBytes) {
          channel::cuda_p2p::Options o;
          o.eagerThreshold = eagerThreshold;
          o.inboxBytes = inboxBytes;
          o.maxCtas = maxCtas;
          o.waitWithKernel = waitWithKernel;
          o.useBulkCopy = useBulkCopy;
          o.sendOrderMinBytes = sendOrderMinBytes;
          o.hostCopyMinBytes = hostCopyMinBytes;
          return channel::cuda_p2p::create(o);
        },
        py::arg("eager_threshold") = defaults.eagerThreshold, py::arg("inbox_bytes") = defaults.inboxBytes,
        py::arg("max_ctas") = defaults.maxCtas, py::arg("wait_with_kernel") = defaults.waitWithKernel,
        py::arg("use_bulk_copy") = defaults.useBulkCopy, py::arg("send_order_min_bytes") = defaults.sendOrderMinBytes,
        py::arg("host_copy_min_bytes") = defaults.hostCopyMinBytes);
  }
  m.def(
      "create_mpt_channel",
      [](int lanes) {
        std::vector<std::shared_ptr<transport::Context>> ctxs;
        std::vector<std::shared_ptr<transport::Listener>> listeners;
        for (int i = 0; i < lanes; ++i) {
          auto c = transport::uv::create();
          listeners.push_back(c->listen("127.0.0.1"));
          ctxs.push_back(std::move(c));
        }
        return channel::mpt::create(std::move(ctxs), std::move(listeners));
      },
      py::arg("lanes") = 4);

  py::class_<PyOutMessage>(m, "OutgoingMessage")
      .def(py::init([](py::bytes metadata) {
             PyOutMessage msg;
             msg.msg.metadata = std::string(metadata);
             return msg;
           }),
           py::arg("metadata") = py::bytes())
      .def("add_payload",
           [](PyOutMessage& self, py::buffer buf, py::bytes metadata) {
             py::buffer_info info = buf.request();
             Message::Payload p;
             p.data = info.ptr;
             p.length = static_cast<size_t>(info.size * info.itemsize);
             p.metadata = std::string(metadata);
             self.msg.payloads.push_back(p);
             self.keep->objects.push_back(std::move(buf));
           },
           py::arg("buffer"), py::arg("metadata") = py::bytes())
      .def("add_tensor",
           [](PyOutMessage& self, uint64_t ptr, uint64_t length, const std::string& deviceType, int deviceIndex,
              uint64_t stream, py::bytes metadata, int dtype, py::object view, py::object targetDevice,
              py::object keep) {
             Message::Tensor t;
             t.buffer = makeBuffer(deviceType, deviceIndex, ptr, stream);
             t.length = length;
             t.metadata = std::string(metadata);
             t.dtype = static_cast<DType>(dtype);
             if (!view.is_none()) {
               auto v = view.cast<std::tuple<int64_t, int64_t, int64_t, int64_t>>();
               StridedView sv;
               sv.dtype = t.dtype;
               sv.rows = std::get<0>(v);
               sv.cols = std::get<1>(v);
               sv.rowStride = std::get<2>(v);
               sv.colStride = std::get<3>(v);
               t.view = sv;
             }
             if (!targetDevice.is_none()) t.targetDevice = parseDevice(targetDevice.cast<std::string>());
             self.msg.tensors.push_back(t);
             if (!keep.is_none()) self.keep->objects.push_back(std::move(keep));
           },
           py::arg("ptr"), py::arg("length"), py::arg("device_type"), py::arg("device_index"), py::arg("stream") = 0,
           py::arg("metadata") = py::bytes(), py::arg("dtype") = 0, py::arg("view") = py::none(),
           py::arg("target_device") = py::none(), py::arg("keep") = py::none());

  py::class_<PyAllocation>(m, "Allocation")
      .def(py::init<>())
      .def("add_payload",
           [](PyAllocation& self, py::buffer buf) {
             py::buffer_info info = buf.request(true);
             self.alloc.payloads.push_back({info.ptr});
             self.keep->objects.push_back(std::move(buf));
           })
      .def("add_tensor",
           [](PyAllocation& self, uint64_t ptr, const std::string& deviceType, int deviceIndex, uint64_t stream,
              py::object castTo, int sourceDtype, py::object keep) {
             Allocation::Tensor t;
             t.buffer = makeBuffer(deviceType, deviceIndex, ptr, stream);
             if (!castTo.is_none()) {
               t.castTo = static_cast<DType>(castTo.cast<int>());
               t.sourceDtype = static_cast<DType>(sourceDtype);
             }
             self.alloc.tensors.push_back(t);
             if (!keep.is_none()) self.keep->objects.push_back(std::move(keep));
           },
           py::arg("ptr"), py::arg("device_type"), py::arg("device_index"), py::arg("stream") = 0,
           py::arg("cast_to") = py::none(), py::arg("source_dtype") = 0, py::arg("keep") = py::none());

  py::class_<Pipe, std::shared_ptr<Pipe>>(m, "Pipe")
      .def("write",
           [](Pipe& self, PyOutMessage& msg, py::function fn) {
             auto cb = wrapCallback<std::string>(std::move(fn), msg.keep);
             Message copy = msg.msg;
             py::gil_scoped_release nogil;
             self.write(std::move(copy), [cb](const Error& e) { cb(errorString(e)); });
           })
      .def("read_descriptor",
           [](Pipe& self, py::function fn) {
             auto holder = std::make_shared<PyKeepAlive>();
             holder->objects.push_back(std::move(fn));
             py::gil_scoped_release nogil;
             self.readDescriptor([holder](const Error& e, Descriptor d) {
               CallbackGil gil;
               try {
                 py::function f = py::reinterpret_borrow<py::function>(holder->objects[0]);
                 f(errorString(e), descriptorToDict(d));
               } catch (py::error_already_set& err) {
                 err.discard_as_unraisable("tensorpipe_b200 read_descriptor callback");
               }
             });
           })
      .def("read",
           [](Pipe& self, PyAllocation& alloc, py::function fn) {
             auto cb = wrapCallback<std::string>(std::move(fn), alloc.keep);
             Allocation copy = alloc.alloc;
             py::gil_scoped_release nogil;
             self.read(std::move(copy), [cb](const Error& e) { cb(errorString(e)); });
           })
      .def("remote_name", [](Pipe& self) { return self.getRemoteName(); })
      .def("set_timeouts",
           [](Pipe& self, int64_t writeMs, int64_t readMs, int64_t descriptorMs) {
             PipeTimeouts t;
             t.write = std::chrono::milliseconds(writeMs);
             t.read = std::chrono::milliseconds(readMs);
             t.descriptor = std::chrono::milliseconds(descriptorMs);
             self.setTimeouts(t);
           },
           py::arg("write_ms") = 0, py::arg("read_ms") = 0, py::arg("descriptor_ms") = 0,
           "Deadlines for operations issued from now on (0 = wait forever); a missed one fails the pipe with 'timeout'.")
      .def("transport_name", &Pipe::transportName, py::call_guard<py::gil_scoped_release>())
      .def("channel_supports_layouts",
           [](Pipe& self, const std::string& local, const std::string& remote) {
             Device l = parseDevice(local), r = parseDevice(remote);
             py::gil_scoped_release nogil;
             return self.channelSupportsLayouts(l, r);
           })
      .def("close", [](Pipe& self) {
        py::gil_scoped_release nogil;
        self.close();
      });

  py::class_<Listener, std::shared_ptr<Listener>>(m, "Listener")
      .def("accept",
           [](Listener& self, py::function fn) {
             auto holder = std::make_shared<PyKeepAlive>();
             holder->objects.push_back(std::move(fn));
             py::gil_scoped_release nogil;
             self.accept([holder](const Error& e, std::shared_ptr<Pipe> p) {
               CallbackGil gil;
               try {
                 py::function f = py::reinterpret_borrow<py::function>(holder->objects[0]);
                 f(errorString(e), p);
               } catch (py::error_already_set& err) {
                 err.discard_as_unraisable("tensorpipe_b200 accept callback");
               }
             });
           })
      .def("url", [](Listener& self, const std::string& t) { return self.url(t); })
      .def("addresses", [](Listener& self) { return self.addresses(); })
      .def("close", [](Listener& self) {
        py::gil_scoped_release nogil;
        self.close();
      });

  py::class_<Context, std::shared_ptr<Context>>(m, "Context")
      .def(py::init([](const std::string& name) { return std::make_shared<Context>(ContextOptions().name(name)); }),
           py::arg("name") = "")
      .def("register_transport", &Context::registerTransport)
      .def("register_channel", &Context::registerChannel)
      .def("listen", [](Context& self, const std::vector<std::string>& urls) { return self.listen(urls); })
      .def("connect",
           [](Context& self, const std::string& url, const std::string& remoteName) {
             return self.connect(url, PipeOptions().remoteName(remoteName));
           },
           py::arg("url"), py::arg("remote_name") = "")
      .def("stats",
           [](Context& self) {
             ContextStats s = self.stats();
             py::dict d;
             d["messages_written"] = s.messagesWritten;
             d["messages_read"] = s.messagesRead;
             d["payload_bytes_written"] = s.payloadBytesWritten;
             d["payload_bytes_read"] = s.payloadBytesRead;
             d["tensor_bytes_sent"] = s.tensorBytesSent;
             d["tensor_bytes_received"] = s.tensorBytesReceived;
             d["pipes_created"] = s.pipesCreated;
             d["bytes_per_channel"] = s.bytesPerChannel;
             d["kernel_launches"] = kernels::launchCount();
             return d;
           })
      .def("close", [](Context& self) {
        py::gil_scoped_release nogil;
        self.close();
      })
      .def("join", [](Context& self) {
        py::gil_scoped_release nogil;
        self.join();
      });

  m.def("kernel_launch_count", &kernels::launchCount);
  m.def("trace_enable", &traceEnable, py::arg("path"),
        "Start recording pipe / channel / kernel-launch events; trace_dump() writes chrome://tracing JSON.");
  m.def("trace_disable", &traceDisable);
  m.def("trace_dump", &traceDump, py::arg("path") = "");
  m.def("trace_event_count", &traceEventCount);
  // Direct access to the push/pack kernel for tests and tools: copy byte ranges between device
  // addresses on the current device with one launch; optionally publish a completion flag
  // (then `counter_ptr` must point to a zeroed 32-bit word in device memory).
  m.def(
      "launch_push",
      [](const std::vector<std::tuple<uint64_t, uint64_t, uint64_t>>& items, uint64_t stream, bool useBulk,
         uint64_t flagPtr, uint32_t flagValue, uint64_t counterPtr) {
        kernels::PushPlan plan;
        for (const auto& it : items) {
          kernels::CopyItem c;
          c.src = reinterpret_cast<const void*>(std::get<0>(it));
          c.dst = reinterpret_cast<void*>(std::get<1>(it));
          c.srcBytes = std::get<2>(it);
          kernels::appendToPlan(plan, c, useBulk);
        }
        if (plan.entries.empty() && flagPtr == 0) return 0;
        int dev = 0;
        cudaGetDevice(&dev);
        int sms = 1;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        return kernels::launchPush(plan, reinterpret_cast<cudaStream_t>(stream), sms,
                                   reinterpret_cast<uint32_t*>(flagPtr), flagValue,
                                   reinterpret_cast<uint32_t*>(counterPtr), nullptr);
      },
      py::arg("items"), py::arg("stream") = 0, py::arg("use_bulk") = true, py::arg("flag_ptr") = 0,
      py::arg("flag_value") = 0, py::arg("counter_ptr") = 0);

  // ---- native benchmark engine ----
  py::class_<tools::PhaseResult>(m, "PhaseResult")
      .def_readonly("device_ms", &tools::PhaseResult::deviceMs)
      .def_readonly("host_ms", &tools::PhaseResult::hostMs)
      .def_readonly("mismatches", &tools::PhaseResult::mismatches)
      .def_readonly("kernel_launches", &tools::PhaseResult::kernelLaunches);
  py::class_<tools::RingBench>(m, "RingBench")
      .def(py::init([](int device, bool useShm, bool useBulkCopy, bool waitWithKernel, size_t eagerThreshold,
                       int maxCtas, size_t maxBytes, const std::string& channel) {
             tools::RingBenchOptions o;
             o.device = device;
             o.useShm = useShm;
             o.useBulkCopy = useBulkCopy;
             o.waitWithKernel = waitWithKernel;
             o.eagerThreshold = eagerThreshold;
             o.maxCtas = maxCtas;
             o.maxBytes = maxBytes;
             o.channel = channel;
             py::gil_scoped_release nogil;
             return std::make_unique<tools::RingBench>(o);
           }),
           py::arg("device") = 0, py::arg("use_shm") = true, py::arg("use_bulk_copy") = true,
           py::arg("wait_with_kernel") = false, py::arg("eager_threshold") = 64 * 1024, py::arg("max_ctas") = 0,
           py::arg("max_bytes") = 1ull << 30, py::arg("channel") = "cuda_p2p")
      .def("listen_url", &tools::RingBench::listenUrl)
      .def("connect", &tools::RingBench::connect, py::call_guard<py::gil_scoped_release>())
      .def("run_stream", &tools::RingBench::runStream, py::arg("bytes"), py::arg("steps"), py::arg("depth") = 2,
           py::arg("verify") = false, py::call_guard<py::gil_scoped_release>())
      .def("run_latency", &tools::RingBench::runLatency, py::arg("bytes"), py::arg("laps"), py::arg("rank") = 0,
           py::arg("world") = 1, py::call_guard<py::gil_scoped_release>())
      .def("run_end_to_end", &tools::RingBench::runEndToEnd, py::arg("bytes"), py::arg("steps"), py::arg("verify") = false,
           py::call_guard<py::gil_scoped_release>())
      .def("connect_mesh", &tools::RingBench::connectMesh, py::call_guard<py::gil_scoped_release>())
      .def(
          "run_mixed_mesh",
          [](tools::RingBench& self, int steps, uint64_t seed) {
            uint64_t bytes = 0;
            tools::PhaseResult r;
            {
              py::gil_scoped_release nogil;
              r = self.runMixedMesh(steps, seed, &bytes);
            }
            return py::make_tuple(r, bytes);
          },
          py::arg("steps"), py::arg("seed") = 1)
      .def(
          "run_mixed",
          [](tools::RingBench& self, int steps, uint64_t seed, bool verify) {
            uint64_t bytes = 0;
            tools::PhaseResult r;
            {
              py::gil_scoped_release nogil;
              r = self.runMixed(steps, seed, &bytes, verify);
            }
            return py::make_tuple(r, bytes);
          },
          py::arg("steps"), py::arg("seed") = 1, py::arg("verify") = false);
}
