// Native CUDA-graph executor for the decode loop.
//
//   begin_capture(stream)  -> everything launched on `stream` until end_capture() is recorded, not run
//   end_capture(stream)    -> the captured graph is checked (kernel nodes only: a memcpy / memset / host node in
//                             a decode graph would serialise against other work and is rejected unless allowed),
//                             its kernel -> kernel edges INTO kernels of this library are rewritten as PROGRAMMATIC
//                             dependencies (so the next
//                             kernel's prologue -- barrier init, TMEM allocation, descriptor prefetch -- overlaps
//                             the previous kernel's tail; every kernel of this library executes
//                             griddepcontrol.wait before touching global data), and an executable is instantiated
//   launch(exec, stream)   -> one cudaGraphLaunch; any number of replays may be queued back to back
//
// (behavioural spec: src/engine/graph_check.hpp:30-77 kernels-only check, src/engine/graph_pdl.hpp:42-87
//  programmatic edges, src/core/graph.hpp GraphCache of the reference.)
#include <string.h>

#include <vector>

#include "common/common.h"

namespace {

struct GraphExec {
  cudaGraph_t graph = nullptr;
  cudaGraphExec_t exec = nullptr;
  int kernel_nodes = 0;
  int other_nodes = 0;
  int programmatic_edges = 0;
};

// True when the kernel node runs a kernel of this library (namespace dgpp).  Only those execute griddepcontrol.wait
// before they touch global data, so only edges INTO them may become programmatic: CUDA makes the predecessor's writes
// visible to a programmatic dependent at that wait, and a kernel without it could read stale data.
static bool own_kernel(cudaGraphNode_t node) {
  cudaKernelNodeParams kp;
  memset(&kp, 0, sizeof(kp));
  if (cudaGraphKernelNodeGetParams(node, &kp) != cudaSuccess || !kp.func) {
    cudaGetLastError();
    return false;
  }
  const char* name = nullptr;
  if (cudaFuncGetName(&name, kp.func) != cudaSuccess || !name) {
    cudaGetLastError();
    return false;
  }
  return strstr(name, "4dgpp") != nullptr;   // Itanium mangling of namespace dgpp
}

// Rewrites the kernel -> kernel edges of `graph` whose successor is a kernel of this library as programmatic edges;
// returns how many were rewritten.
static int rewrite_pdl_edges(cudaGraph_t graph) {
  int rewritten = 0;
  size_t ne = 0;
  if (cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &ne) != cudaSuccess || !ne) {
    cudaGetLastError();
    return 0;
  }
  std::vector<cudaGraphNode_t> from(ne), to(ne);
  std::vector<cudaGraphEdgeData> data(ne);
  cudaGraphGetEdges_v2(graph, from.data(), to.data(), data.data(), &ne);
  for (size_t e = 0; e < ne; ++e) {
    cudaGraphNodeType tf, tt;
    cudaGraphNodeGetType(from[e], &tf);
    cudaGraphNodeGetType(to[e], &tt);
    if (tf != cudaGraphNodeTypeKernel || tt != cudaGraphNodeTypeKernel) continue;
    if (data[e].type == cudaGraphDependencyTypeProgrammatic) continue;
    if (!own_kernel(to[e])) continue;   // a foreign kernel (NCCL, torch) never executes griddepcontrol.wait
    cudaGraphEdgeData nd;
    memset(&nd, 0, sizeof(nd));
    nd.from_port = cudaGraphKernelNodePortProgrammatic;
    nd.to_port = 0;
    nd.type = cudaGraphDependencyTypeProgrammatic;
    if (cudaGraphRemoveDependencies_v2(graph, &from[e], &to[e], &data[e], 1) != cudaSuccess) {
      cudaGetLastError();
      continue;
    }
    if (cudaGraphAddDependencies_v2(graph, &from[e], &to[e], &nd, 1) != cudaSuccess) {
      cudaGetLastError();
      cudaGraphAddDependencies_v2(graph, &from[e], &to[e], &data[e], 1);  // put the plain edge back
      continue;
    }
    ++rewritten;
  }
  return rewritten;
}

}  // namespace

DGPP_API int dgpp_graph_begin_capture(cudaStream_t st) {
  DGPP_CUDA_OK(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
  return 0;
}

// pdl: rewrite kernel->kernel edges as programmatic.  allow_non_kernel: keep memcpy/memset nodes (debug graphs).
// info_out[0..2] = kernel nodes, other nodes, programmatic edges.
DGPP_API void* dgpp_graph_end_capture(cudaStream_t st, int pdl, int allow_non_kernel, int* info_out) {
  GraphExec* g = new GraphExec();
  if (cudaStreamEndCapture(st, &g->graph) != cudaSuccess || !g->graph) {
    dgpp_set_error("graph: cudaStreamEndCapture failed: %s", cudaGetErrorString(cudaGetLastError()));
    delete g;
    return nullptr;
  }
  size_t n = 0;
  cudaGraphGetNodes(g->graph, nullptr, &n);
  std::vector<cudaGraphNode_t> nodes(n);
  if (n) cudaGraphGetNodes(g->graph, nodes.data(), &n);
  for (size_t i = 0; i < n; ++i) {
    cudaGraphNodeType t;
    cudaGraphNodeGetType(nodes[i], &t);
    if (t == cudaGraphNodeTypeKernel) ++g->kernel_nodes; else ++g->other_nodes;
  }
  if (g->other_nodes && !allow_non_kernel) {
    dgpp_set_error("graph: %d non-kernel node(s) in a decode graph (memcpy / memset / host); use kernels", g->other_nodes);
    cudaGraphDestroy(g->graph);
    delete g;
    return nullptr;
  }
  if (pdl) g->programmatic_edges = rewrite_pdl_edges(g->graph);
  if (cudaGraphInstantiate(&g->exec, g->graph, 0) != cudaSuccess) {
    dgpp_set_error("graph: cudaGraphInstantiate failed: %s", cudaGetErrorString(cudaGetLastError()));
    cudaGraphDestroy(g->graph);
    delete g;
    return nullptr;
  }
  if (info_out) {
    info_out[0] = g->kernel_nodes;
    info_out[1] = g->other_nodes;
    info_out[2] = g->programmatic_edges;
  }
  return g;
}

// The same edge rewrite on a graph somebody else captured and will instantiate (a framework's graph object that keeps
// its cudaGraph_t until the first replay).  info_out[0..2] = kernel nodes, other nodes, programmatic edges.
DGPP_API int dgpp_graph_pdl_rewrite(void* raw_graph, int* info_out) {
  DGPP_REQUIRE(raw_graph != nullptr, "graph_pdl_rewrite: null graph");
  cudaGraph_t graph = static_cast<cudaGraph_t>(raw_graph);
  size_t n = 0;
  DGPP_CUDA_OK(cudaGraphGetNodes(graph, nullptr, &n));
  std::vector<cudaGraphNode_t> nodes(n);
  if (n) DGPP_CUDA_OK(cudaGraphGetNodes(graph, nodes.data(), &n));
  int kernels = 0, others = 0;
  for (size_t i = 0; i < n; ++i) {
    cudaGraphNodeType t;
    cudaGraphNodeGetType(nodes[i], &t);
    if (t == cudaGraphNodeTypeKernel) ++kernels; else ++others;
  }
  const int edges = rewrite_pdl_edges(graph);
  if (info_out) {
    info_out[0] = kernels;
    info_out[1] = others;
    info_out[2] = edges;
  }
  return 0;
}

DGPP_API int dgpp_graph_launch(void* handle, cudaStream_t st) {
  GraphExec* g = static_cast<GraphExec*>(handle);
  DGPP_REQUIRE(g && g->exec, "graph: launch of an empty handle");
  DGPP_CUDA_OK(cudaGraphLaunch(g->exec, st));
  return 0;
}

DGPP_API int dgpp_graph_destroy(void* handle) {
  GraphExec* g = static_cast<GraphExec*>(handle);
  if (!g) return 0;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Native decode loop: replays one captured decode-step graph `steps` times with at most `inflight` (1..4) steps
// outstanding.  The step graph feeds itself on the device (its last kernel writes the picked ids where its first kernel
// reads the input ids), so the host never sits between two steps.  After every replay the step's picked ids and the
// device status block are copied into a pinned mailbox slot and an event is recorded; the host retires the slots in
// order: ids go to `out[step * b ..]`, rows that produced one of `stop_ids` are marked, a non-zero status code ends the
// loop with an error.  Once every row is marked no further step is launched; steps already in flight are drained and
// their ids dropped.  Returns 0, or -1 with dgpp_last_error() set (status code / CUDA error).
//   d_tokens   device int32 [>= b]: the step graph's token mailbox (input of the next step = output of this one)
//   out        host int32 [steps * b]; row_stop host int32 [b]: index of the step at which the row stopped, or -1
//   steps_run  host int [2]: steps whose ids were delivered to `out`, steps launched (the device state advanced that far)
// (behavioural spec: src/engine/graph_engine.hpp:2860-2995 launch / settle_front with two replays in flight.)
namespace dgpp { DeviceStatus* device_status_ptr(); }

namespace {

struct Mailbox {
  int32_t* host = nullptr;     // pinned [slots][kMaxBatch + 4]
  cudaEvent_t ev[4] = {nullptr, nullptr, nullptr, nullptr};
  int dev = -1;
};
constexpr int kLoopMaxBatch = 512;

static Mailbox* mailbox() {
  static thread_local Mailbox mb;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (mb.host && mb.dev == dev) return &mb;
  if (mb.host) {
    cudaFreeHost(mb.host);
    for (auto& e : mb.ev) if (e) { cudaEventDestroy(e); e = nullptr; }
    mb.host = nullptr;
  }
  if (cudaHostAlloc(reinterpret_cast<void**>(&mb.host), 4 * (kLoopMaxBatch + 4) * sizeof(int32_t), cudaHostAllocDefault) != cudaSuccess)
    return nullptr;
  for (auto& e : mb.ev)
    if (cudaEventCreateWithFlags(&e, cudaEventDisableTiming) != cudaSuccess) return nullptr;
  mb.dev = dev;
  return &mb;
}

}  // namespace

DGPP_API int dgpp_decode_loop(void* graph, const void* d_tokens, int b, int steps, int inflight, const int32_t* stop_ids,
                              int n_stop, int32_t* out, int32_t* row_stop, int* steps_run, cudaStream_t st) {
  GraphExec* g = static_cast<GraphExec*>(graph);
  DGPP_REQUIRE(g && g->exec, "decode_loop: empty graph handle");
  DGPP_REQUIRE(b >= 1 && b <= kLoopMaxBatch && steps >= 0 && inflight >= 1 && inflight <= 4, "decode_loop: bad sizes (b %d inflight %d)",
               b, inflight);
  Mailbox* mb = mailbox();
  DGPP_REQUIRE(mb != nullptr, "decode_loop: pinned mailbox allocation failed");
  dgpp::DeviceStatus* status = dgpp::device_status_ptr();
  DGPP_REQUIRE(status != nullptr, "decode_loop: no status block");
  const int stride = kLoopMaxBatch + 4;
  for (int r = 0; r < b; ++r) row_stop[r] = -1;
  int launched = 0, retired = 0, delivered = 0, live = b;
  bool stop_launching = false;
  while (retired < launched || (!stop_launching && launched < steps)) {
    while (!stop_launching && launched < steps && launched - retired < inflight) {
      const int slot = launched % 4;
      DGPP_CUDA_OK(cudaGraphLaunch(g->exec, st));
      DGPP_CUDA_OK(cudaMemcpyAsync(mb->host + slot * stride, d_tokens, b * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
      DGPP_CUDA_OK(cudaMemcpyAsync(mb->host + slot * stride + kLoopMaxBatch, status, 4 * sizeof(int32_t), cudaMemcpyDeviceToHost, st));
      DGPP_CUDA_OK(cudaEventRecord(mb->ev[slot], st));
      ++launched;
    }
    if (retired < launched) {
      const int slot = retired % 4;
      DGPP_CUDA_OK(cudaEventSynchronize(mb->ev[slot]));
      const int32_t* ids = mb->host + slot * stride;
      const int32_t* stt = ids + kLoopMaxBatch;
      if (stt[0] != 0) {
        cudaStreamSynchronize(st);
        steps_run[0] = delivered;
        steps_run[1] = launched;
        dgpp_set_error("decode_loop: device status code=%d count=%d detail=%d at step %d", stt[0], stt[1], stt[2], retired);
        return -1;
      }
      if (!stop_launching) {
        for (int r = 0; r < b; ++r) {
          out[static_cast<size_t>(retired) * b + r] = ids[r];
          if (row_stop[r] < 0)
            for (int k = 0; k < n_stop; ++k)
              if (ids[r] == stop_ids[k]) { row_stop[r] = retired; --live; break; }
        }
        ++delivered;
        if (live == 0) stop_launching = true;
      }
      ++retired;
    }
  }
  steps_run[0] = delivered;
  steps_run[1] = launched;
  return 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// Bounded host-side waits: a stream or an event is polled with a deadline instead of a blocking synchronize, so a device
// that stopped making progress turns into a return code the caller can act on (fail the engine, report, exit) rather
// than a hung server thread.  Returns 0 = finished, 1 = deadline passed (work still pending), -1 = CUDA error.
// (behavioural spec: src/core/cuda_wait.hpp of the reference.)
#include <chrono>
#include <thread>

static int bounded_poll(cudaError_t (*query)(void*), void* what, int64_t timeout_us) {
  const auto t0 = std::chrono::steady_clock::now();
  int spins = 0;
  for (;;) {
    const cudaError_t e = query(what);
    if (e == cudaSuccess) return 0;
    if (e != cudaErrorNotReady) {
      dgpp_set_error("bounded wait: %s", cudaGetErrorString(e));
      cudaGetLastError();
      return -1;
    }
    const auto us = std::chrono::duration_cast<std::chrono::microseconds>(std::chrono::steady_clock::now() - t0).count();
    if (us >= timeout_us) return 1;
    if (++spins < 2000) continue;                                  // ~first tens of microseconds: pure polling
    std::this_thread::sleep_for(std::chrono::microseconds(us < 2000 ? 20 : 200));
  }
}

DGPP_API int dgpp_stream_wait(cudaStream_t st, int64_t timeout_us) {
  return bounded_poll([](void* s) { return cudaStreamQuery(static_cast<cudaStream_t>(s)); }, st, timeout_us);
}

DGPP_API int dgpp_event_wait(cudaEvent_t ev, int64_t timeout_us) {
  return bounded_poll([](void* e) { return cudaEventQuery(static_cast<cudaEvent_t>(e)); }, ev, timeout_us);
}
