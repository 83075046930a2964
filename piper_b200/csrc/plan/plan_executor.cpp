// Launch-plan executor: replays one rank's dispatch order once per training step.
//
// The plan is built once from the per-device training DAG: for every node its CUDA stream, the earlier nodes whose
// completion it has to wait for (only those that ran on another stream), and a label.  One cudaEvent_t per node
// is created with the plan and re-recorded every step, so a step allocates no events.  run(callback) walks the
// plan: make the node's stream current (for PyTorch and for this library's kernels), enqueue the event waits,
// open an NVTX range, call back into Python for the node's body, record the node's event.  With timing enabled
// every node is bracketed by two timing events and elapsed() returns the device time per node after the step.
//
// The reference interprets its DAG in a Python loop with a `match` per node and creates its events per step
// (src/executors.py:571-1003); here only the bodies of the nodes are Python.
#include <c10/cuda/CUDAStream.h>
#include <cuda_runtime.h>
#include <nvtx3/nvToolsExt.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <stdexcept>
#include <string>
#include <vector>

namespace py = pybind11;

namespace {

void check(cudaError_t e, const char* what) {
  if (e != cudaSuccess) throw std::runtime_error(std::string("plan executor: ") + what + ": " + cudaGetErrorString(e));
}

struct Node {
  int stream = 0;
  std::vector<int> waits;
  std::string label;
};

class PlanExecutor {
 public:
  PlanExecutor(int device, std::vector<uintptr_t> streams, std::vector<int> node_stream,
               std::vector<std::vector<int>> node_waits, std::vector<std::string> labels, bool nvtx)
      : device_(device), nvtx_(nvtx) {
    const size_t n = node_stream.size();
    if (node_waits.size() != n || labels.size() != n) throw std::invalid_argument("plan executor: ragged plan");
    for (uintptr_t s : streams) streams_.push_back(reinterpret_cast<cudaStream_t>(s));
    nodes_.resize(n);
    for (size_t i = 0; i < n; ++i) {
      if (node_stream[i] < 0 || node_stream[i] >= static_cast<int>(streams_.size()))
        throw std::invalid_argument("plan executor: stream index out of range");
      for (int w : node_waits[i])
        if (w < 0 || w >= static_cast<int>(i)) throw std::invalid_argument("plan executor: a node waits for a later node");
      nodes_[i].stream = node_stream[i];
      nodes_[i].waits = std::move(node_waits[i]);
      nodes_[i].label = std::move(labels[i]);
    }
    check(cudaSetDevice(device_), "cudaSetDevice");
    done_.resize(n);
    for (size_t i = 0; i < n; ++i) check(cudaEventCreateWithFlags(&done_[i], cudaEventDisableTiming), "cudaEventCreate");
  }

  ~PlanExecutor() {
    for (cudaEvent_t e : done_) cudaEventDestroy(e);
    for (cudaEvent_t e : t0_) cudaEventDestroy(e);
    for (cudaEvent_t e : t1_) cudaEventDestroy(e);
  }

  void set_timing(bool on) {
    timing_ = on;
    if (on && t0_.empty()) {
      t0_.resize(nodes_.size());
      t1_.resize(nodes_.size());
      for (size_t i = 0; i < nodes_.size(); ++i) {
        check(cudaEventCreate(&t0_[i]), "cudaEventCreate");
        check(cudaEventCreate(&t1_[i]), "cudaEventCreate");
      }
    }
  }

  // Bound on how far the host may run ahead of the device: before node i is issued the host waits until node
  // i - n has completed (0: no bound).  Memory that a node frees after use on a second stream returns to the
  // caching allocator only when the device has passed that use, so an unbounded host keeps more blocks alive.
  void set_max_ahead(int n) { max_ahead_ = n < 0 ? 0 : n; }

  // callback(i) runs the body of node i on the current stream.
  void run(const py::function& callback) {
    const c10::cuda::CUDAStream before = c10::cuda::getCurrentCUDAStream(device_);
    timed_ = timing_;
    try {
      for (size_t i = 0; i < nodes_.size(); ++i) {
        const Node& nd = nodes_[i];
        cudaStream_t s = streams_[nd.stream];
        if (max_ahead_ > 0 && i >= static_cast<size_t>(max_ahead_)) {
          py::gil_scoped_release release;
          check(cudaEventSynchronize(done_[i - max_ahead_]), "cudaEventSynchronize");
        }
        c10::cuda::setCurrentCUDAStream(c10::cuda::getStreamFromExternal(s, device_));
        for (int w : nd.waits) check(cudaStreamWaitEvent(s, done_[w], 0), "cudaStreamWaitEvent");
        if (nvtx_) nvtxRangePushA(nd.label.c_str());
        if (timed_) check(cudaEventRecord(t0_[i], s), "cudaEventRecord");
        try {
          callback(i);
        } catch (...) {
          if (nvtx_) nvtxRangePop();
          throw;
        }
        if (timed_) check(cudaEventRecord(t1_[i], s), "cudaEventRecord");
        check(cudaEventRecord(done_[i], s), "cudaEventRecord");
        if (nvtx_) nvtxRangePop();
      }
    } catch (...) {
      c10::cuda::setCurrentCUDAStream(before);
      throw;
    }
    c10::cuda::setCurrentCUDAStream(before);
  }

  // Device milliseconds of every node of the last timed step (synchronises with the last node).
  std::vector<float> elapsed() {
    std::vector<float> out(nodes_.size(), 0.f);
    if (!timed_) return out;
    for (size_t i = 0; i < nodes_.size(); ++i) {
      check(cudaEventSynchronize(t1_[i]), "cudaEventSynchronize");
      check(cudaEventElapsedTime(&out[i], t0_[i], t1_[i]), "cudaEventElapsedTime");
    }
    return out;
  }

  size_t size() const { return nodes_.size(); }
  size_t num_waits() const {
    size_t n = 0;
    for (const Node& nd : nodes_) n += nd.waits.size();
    return n;
  }

 private:
  int device_;
  bool nvtx_;
  bool timing_ = false, timed_ = false;
  int max_ahead_ = 0;
  std::vector<cudaStream_t> streams_;
  std::vector<Node> nodes_;
  std::vector<cudaEvent_t> done_, t0_, t1_;
};

}  // namespace

PYBIND11_MODULE(piper_plan, m) {
  m.doc() = "launch-plan executor of piper_b200 (see csrc/plan/plan_executor.cpp)";
  py::class_<PlanExecutor>(m, "PlanExecutor")
      .def(py::init<int, std::vector<uintptr_t>, std::vector<int>, std::vector<std::vector<int>>,
                    std::vector<std::string>, bool>(),
           py::arg("device"), py::arg("streams"), py::arg("node_stream"), py::arg("node_waits"), py::arg("labels"),
           py::arg("nvtx") = false)
      .def("run", &PlanExecutor::run)
      .def("set_timing", &PlanExecutor::set_timing)
      .def("set_max_ahead", &PlanExecutor::set_max_ahead)
      .def("elapsed", &PlanExecutor::elapsed)
      .def("__len__", &PlanExecutor::size)
      .def_property_readonly("num_waits", &PlanExecutor::num_waits);
}
