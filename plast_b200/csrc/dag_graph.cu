// A scheduler DAG as one CUDA graph: the kernels of every node are recorded once by stream capture
// and replayed with a single launch. Small graphs (the 1024 x 1024 add -> relu -> row-sum case)
// are bound by the ~4 us a kernel launch costs in a stream, not by HBM; a replayed graph runs the
// same kernels back to back at 2-3 us each. The reference's JIT mode re-executes a cached DAG
// object node by node (src/scheduler/scheduler.c:17-27, src/scheduler/jit.c:70-80): that cached
// object is what gets captured here, on the same tensors.
#include "common.cuh"
#include "plast_b200_graph.h"

#include <dlfcn.h>
#include <string.h>

struct PlastDagGraph {
  cudaGraph_t graph;
  cudaGraphExec_t exec;
  int kernels; // kernel nodes in the graph, for the launch counter
};

namespace pb {
namespace {

// True when fn is a function of THIS shared library. Only such kernels go to the library stream
// and can be captured; a foreign kernel (the reference's matmul / conv objects launch on the
// legacy default stream and synchronise the device) would silently drop out of the graph.
bool ours(const void *fn) {
  Dl_info mine = {}, theirs = {};
  if (!fn || !dladdr((const void *)&plast_b200_dag_capture, &mine) || !dladdr(fn, &theirs)) return false;
  return mine.dli_fbase == theirs.dli_fbase;
}

} // namespace
} // namespace pb

using namespace pb;

extern "C" {

PlastDagGraph *plast_b200_dag_capture(DAG *dag, int backward) {
  begin_call();
  if (!dag || !dag->nodes || dag->count == 0) {
    set_error(PLAST_B200_ERR_NULL, "dag capture: empty DAG");
    return nullptr;
  }
  for (u32 i = 0; i < dag->count; ++i) {
    const Node *n = dag->nodes[i];
    const bool fwd_ok = n && (backward == 1 || ours((const void *)n->op.cuda_forward));
    const bool bwd_ok = n && (backward == 0 || ours((const void *)n->op.cuda_backward));
    if (!n || !n->output || n->output->device != CUDA || !fwd_ok || !bwd_ok) {
      set_error(PLAST_B200_ERR_UNSUPPORTED, "dag capture: node %u is not a CUDA node of this library", i);
      return nullptr;
    }
  }
  Workspace ws;
  if (!get_workspace(&ws)) return nullptr; // allocated now, not in the middle of the capture
  cudaStream_t capture_stream = nullptr;
  PB_CUDA_RET(cudaStreamCreateWithFlags(&capture_stream, cudaStreamNonBlocking), nullptr);
  void *const user_stream = plast_b200_get_stream();
  // Relaxed mode: calls that are not stream work (a run-time compile loading its module, the
  // occupancy queries) stay legal while capturing. The per-op device synchronise is not.
  const bool user_sync = sync_enabled();
  plast_b200_set_sync(0);
  plast_b200_set_stream(capture_stream);
  cudaGraph_t graph = nullptr;
  bool ok = cudaStreamBeginCapture(capture_stream, cudaStreamCaptureModeRelaxed) == cudaSuccess;
  if (!ok) set_error(PLAST_B200_ERR_CUDA, "dag capture: cannot begin stream capture");
  int failed_node = -1;
  char failed_message[256] = "";
  if (ok) {
    // mode 0: forward pass; 1: backward pass; 2: forward pass followed by the backward pass
    for (int pass = 0; pass < 2; ++pass) {
      const bool run_backward = pass == 1;
      if ((run_backward && backward == 0) || (!run_backward && backward == 1)) continue;
      for (u32 k = 0; k < dag->count && failed_node < 0; ++k) {
        Node *n = dag->nodes[run_backward ? dag->count - 1 - k : k];
        if (run_backward) n->op.cuda_backward(n->inputs, n->output, n->params);
        else n->op.cuda_forward((const Tensor **)n->inputs, n->output, n->params);
        if (plast_b200_last_error() != PLAST_B200_OK) {
          failed_node = (int)k;
          strncpy(failed_message, plast_b200_last_error_message(), sizeof(failed_message) - 1);
        }
      }
    }
    const cudaError_t e = cudaStreamEndCapture(capture_stream, &graph);
    if (e != cudaSuccess || !graph) {
      ok = false;
      cudaGetLastError();
      begin_call();
      set_error(PLAST_B200_ERR_CUDA, "dag capture: stream capture failed: %s", cudaGetErrorString(e));
    }
  }
  plast_b200_set_stream(user_stream);
  plast_b200_set_sync(user_sync ? 1 : 0);
  cudaStreamDestroy(capture_stream);
  if (ok && failed_node >= 0) {
    ok = false;
    begin_call();
    set_error(PLAST_B200_ERR_UNSUPPORTED, "dag capture: node %d failed while recording: %s", failed_node, failed_message);
  }
  if (!ok) {
    if (graph) cudaGraphDestroy(graph);
    return nullptr;
  }
  PlastDagGraph *g = new PlastDagGraph();
  g->graph = graph;
  g->exec = nullptr;
  g->kernels = 0;
  if (cudaGraphInstantiate(&g->exec, graph, 0) != cudaSuccess) {
    cudaGetLastError();
    cudaGraphDestroy(graph);
    delete g;
    begin_call();
    set_error(PLAST_B200_ERR_CUDA, "dag capture: the recorded graph could not be instantiated");
    return nullptr;
  }
  size_t n_nodes = 0;
  if (cudaGraphGetNodes(graph, nullptr, &n_nodes) == cudaSuccess && n_nodes > 0) {
    cudaGraphNode_t *nodes = new cudaGraphNode_t[n_nodes];
    if (cudaGraphGetNodes(graph, nodes, &n_nodes) == cudaSuccess)
      for (size_t i = 0; i < n_nodes; ++i) {
        cudaGraphNodeType t;
        if (cudaGraphNodeGetType(nodes[i], &t) == cudaSuccess && t == cudaGraphNodeTypeKernel) ++g->kernels;
      }
    delete[] nodes;
  }
  begin_call();
  note_kernel("dag_graph_capture");
  return g;
}

void plast_b200_dag_replay(PlastDagGraph *g) {
  begin_call();
  if (!g || !g->exec) {
    set_error(PLAST_B200_ERR_NULL, "dag replay: no graph");
    return;
  }
  PB_CUDA(cudaGraphLaunch(g->exec, stream()));
  count_launch(g->kernels);
  note_kernel("dag_graph_replay");
  end_call();
}

int plast_b200_dag_graph_kernels(const PlastDagGraph *g) { return g ? g->kernels : 0; }

void plast_b200_dag_graph_release(PlastDagGraph *g) {
  if (!g) return;
  if (g->exec) cudaGraphExecDestroy(g->exec);
  if (g->graph) cudaGraphDestroy(g->graph);
  delete g;
}

} // extern "C"
