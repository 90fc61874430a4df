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
  if (pdl) {
    size_t ne = 0;
    if (cudaGraphGetEdges_v2(g->graph, nullptr, nullptr, nullptr, &ne) == cudaSuccess && ne) {
      std::vector<cudaGraphNode_t> from(ne), to(ne);
      std::vector<cudaGraphEdgeData> data(ne);
      cudaGraphGetEdges_v2(g->graph, from.data(), to.data(), data.data(), &ne);
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
        if (cudaGraphRemoveDependencies_v2(g->graph, &from[e], &to[e], &data[e], 1) != cudaSuccess) {
          cudaGetLastError();
          continue;
        }
        if (cudaGraphAddDependencies_v2(g->graph, &from[e], &to[e], &nd, 1) != cudaSuccess) {
          cudaGetLastError();
          cudaGraphAddDependencies_v2(g->graph, &from[e], &to[e], &data[e], 1);  // put the plain edge back
          continue;
        }
        ++g->programmatic_edges;
      }
    } else {
      cudaGetLastError();
    }
  }
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
