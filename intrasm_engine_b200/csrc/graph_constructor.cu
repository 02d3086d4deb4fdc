// Native CUDA-graph constructor behind the C ABI (host code only).
//
// Builds ONE cudaGraph_t out of work that callers enqueue on several registered streams:
// every registered stream has a "last activity" node; a bracketed library call on a
// stream is captured straight into the graph behind that node
// (cudaStreamBeginCaptureToGraph), event record / wait nodes and joins are added
// explicitly, and the finished graph is instantiated and launched.  Two independent
// chains under one root are what lets the hardware co-schedule a sparse and a dense
// kernel — the baseline the fused kernel is compared with.
//
// Replaces CudaGraphWrapper / CUDAGraphConstructor / CUDAExperimentalGraphConstructor
// (intrasm_engine/common/include/helper_CUDAGraphConstructor.cu.h:106-166, :268-388,
// :406-486) and combineCUDAGraphs (helper_cuda_graph.cu.h:34-62).  Differences: the tail
// of a captured segment is taken from cudaStreamGetCaptureInfo (the capture's current
// dependency set) instead of re-scanning all graph edges after every capture; a segment
// that ends in several leaves is closed with an empty node; errors are returned as
// status codes instead of C++ exceptions; the instantiated executable can be re-launched
// without re-instantiation.
#include <cstdio>
#include <map>
#include <vector>

#include "common.cuh"

namespace {

struct Constructor {
  cudaGraph_t graph = nullptr;
  cudaGraphNode_t root = nullptr;
  cudaGraphExec_t exec = nullptr;
  bool owned = true;  // false once the graph was added to another graph as a child
  std::map<cudaStream_t, cudaGraphNode_t> last;  // last activity per registered stream
  cudaStream_t capturing = nullptr;
  bool is_capturing = false;
};

#define IEX_CUDA(expr)                                   \
  do {                                                   \
    cudaError_t e_ = (expr);                             \
    if (e_ != cudaSuccess) return static_cast<int>(e_);  \
  } while (0)

Constructor* as_ctor(void* h) { return static_cast<Constructor*>(h); }

int last_of(Constructor* c, cudaStream_t s, cudaGraphNode_t* out) {
  auto it = c->last.find(s);
  if (it == c->last.end()) return IEX_ERR_BAD_ARG;  // stream was never registered
  *out = it->second;
  return IEX_OK;
}

}  // namespace

extern "C" void* iex_graph_create(void) {
  Constructor* c = new Constructor();
  if (cudaGraphCreate(&c->graph, 0) != cudaSuccess ||
      cudaGraphAddEmptyNode(&c->root, c->graph, nullptr, 0) != cudaSuccess) {
    if (c->graph) cudaGraphDestroy(c->graph);
    delete c;
    return nullptr;
  }
  return c;
}

extern "C" int iex_graph_destroy(void* h) {
  Constructor* c = as_ctor(h);
  if (!c) return IEX_ERR_BAD_ARG;
  if (c->exec) cudaGraphExecDestroy(c->exec);
  if (c->owned && c->graph) cudaGraphDestroy(c->graph);
  delete c;
  return IEX_OK;
}

extern "C" int iex_graph_register_stream(void* h, void* stream) {
  Constructor* c = as_ctor(h);
  if (!c) return IEX_ERR_BAD_ARG;
  c->last[static_cast<cudaStream_t>(stream)] = c->root;
  return IEX_OK;
}

extern "C" int iex_graph_add_event_record_node(void* h, void* event, void* stream) {
  Constructor* c = as_ctor(h);
  if (!c || !event) return IEX_ERR_BAD_ARG;
  cudaGraphNode_t dep, node;
  int st = last_of(c, static_cast<cudaStream_t>(stream), &dep);
  if (st) return st;
  IEX_CUDA(cudaGraphAddEventRecordNode(&node, c->graph, &dep, 1, static_cast<cudaEvent_t>(event)));
  c->last[static_cast<cudaStream_t>(stream)] = node;
  return IEX_OK;
}

extern "C" int iex_graph_add_stream_wait_event_node(void* h, void* stream, void* event) {
  Constructor* c = as_ctor(h);
  if (!c || !event) return IEX_ERR_BAD_ARG;
  cudaGraphNode_t dep, node;
  int st = last_of(c, static_cast<cudaStream_t>(stream), &dep);
  if (st) return st;
  IEX_CUDA(cudaGraphAddEventWaitNode(&node, c->graph, &dep, 1, static_cast<cudaEvent_t>(event)));
  c->last[static_cast<cudaStream_t>(stream)] = node;
  return IEX_OK;
}

// One empty node that depends on the last activity of every stream in `streams` (and of
// dst_stream itself); it becomes dst_stream's last activity.
extern "C" int iex_graph_join(void* h, void* const* streams, int count, void* dst_stream) {
  Constructor* c = as_ctor(h);
  if (!c || count < 0 || (count > 0 && !streams)) return IEX_ERR_BAD_ARG;
  std::vector<cudaGraphNode_t> deps;
  cudaGraphNode_t n;
  int st = last_of(c, static_cast<cudaStream_t>(dst_stream), &n);
  if (st) return st;
  deps.push_back(n);
  for (int i = 0; i < count; ++i) {
    st = last_of(c, static_cast<cudaStream_t>(streams[i]), &n);
    if (st) return st;
    bool dup = false;
    for (cudaGraphNode_t d : deps) dup |= (d == n);
    if (!dup) deps.push_back(n);
  }
  cudaGraphNode_t join;
  IEX_CUDA(cudaGraphAddEmptyNode(&join, c->graph, deps.data(), deps.size()));
  c->last[static_cast<cudaStream_t>(dst_stream)] = join;
  return IEX_OK;
}

// Everything enqueued on `stream` between capture_begin and capture_end becomes nodes of
// the graph, behind the stream's last activity.
extern "C" int iex_graph_capture_begin(void* h, void* stream) {
  Constructor* c = as_ctor(h);
  if (!c || c->is_capturing) return IEX_ERR_BAD_ARG;
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  cudaGraphNode_t dep;
  int st = last_of(c, s, &dep);
  if (st) return st;
  IEX_CUDA(cudaStreamBeginCaptureToGraph(s, c->graph, &dep, nullptr, 1,
                                         cudaStreamCaptureModeThreadLocal));
  c->capturing = s;
  c->is_capturing = true;
  return IEX_OK;
}

extern "C" int iex_graph_capture_end(void* h, void* stream) {
  Constructor* c = as_ctor(h);
  cudaStream_t s = static_cast<cudaStream_t>(stream);
  if (!c || !c->is_capturing || c->capturing != s) return IEX_ERR_BAD_ARG;
  // The capture's current dependency set = the leaves of what was just recorded.
  cudaStreamCaptureStatus status;
  const cudaGraphNode_t* deps = nullptr;
  size_t ndeps = 0;
  cudaError_t e = cudaStreamGetCaptureInfo_v2(s, &status, nullptr, nullptr, &deps, &ndeps);
  std::vector<cudaGraphNode_t> leaves;
  if (e == cudaSuccess && status == cudaStreamCaptureStatusActive)
    leaves.assign(deps, deps + ndeps);
  cudaGraph_t g = nullptr;
  cudaError_t e2 = cudaStreamEndCapture(s, &g);
  c->is_capturing = false;
  c->capturing = nullptr;
  if (e != cudaSuccess) return static_cast<int>(e);
  if (e2 != cudaSuccess) return static_cast<int>(e2);
  if (leaves.size() == 1) {
    c->last[s] = leaves[0];
  } else if (leaves.size() > 1) {
    cudaGraphNode_t join;
    IEX_CUDA(cudaGraphAddEmptyNode(&join, c->graph, leaves.data(), leaves.size()));
    c->last[s] = join;
  }  // nothing captured: the last activity stays what it was
  return IEX_OK;
}

extern "C" int iex_graph_instantiate(void* h) {
  Constructor* c = as_ctor(h);
  if (!c || c->is_capturing) return IEX_ERR_BAD_ARG;
  if (c->exec) return IEX_ERR_BAD_ARG;  // destroy the previous executable first
  IEX_CUDA(cudaGraphInstantiate(&c->exec, c->graph, 0));
  return IEX_OK;
}

extern "C" int iex_graph_launch(void* h, void* stream) {
  Constructor* c = as_ctor(h);
  if (!c || !c->exec) return IEX_ERR_BAD_ARG;
  IEX_CUDA(cudaGraphLaunch(c->exec, static_cast<cudaStream_t>(stream)));
  return IEX_OK;
}

extern "C" int iex_graph_exec_destroy(void* h) {
  Constructor* c = as_ctor(h);
  if (!c || !c->exec) return IEX_ERR_BAD_ARG;
  IEX_CUDA(cudaGraphExecDestroy(c->exec));
  c->exec = nullptr;
  return IEX_OK;
}

extern "C" int iex_graph_node_count(void* h, long long* nodes, long long* edges) {
  Constructor* c = as_ctor(h);
  if (!c) return IEX_ERR_BAD_ARG;
  size_t n = 0, m = 0;
  IEX_CUDA(cudaGraphGetNodes(c->graph, nullptr, &n));
  IEX_CUDA(cudaGraphGetEdges(c->graph, nullptr, nullptr, &m));
  if (nodes) *nodes = static_cast<long long>(n);
  if (edges) *edges = static_cast<long long>(m);
  return IEX_OK;
}

extern "C" int iex_graph_dump(void* h, const char* path) {
  Constructor* c = as_ctor(h);
  if (!c || !path) return IEX_ERR_BAD_ARG;
  IEX_CUDA(cudaGraphDebugDotPrint(c->graph, path, cudaGraphDebugDotFlagsVerbose));
  return IEX_OK;
}

// Adds `child`'s graph to `h` as a child-graph node behind `h`'s root.  The child graph is
// cloned into the parent by the runtime; the child constructor stays usable.
extern "C" int iex_graph_add_child(void* h, void* child) {
  Constructor* c = as_ctor(h);
  Constructor* ch = as_ctor(child);
  if (!c || !ch || c == ch) return IEX_ERR_BAD_ARG;
  cudaGraphNode_t node;
  IEX_CUDA(cudaGraphAddChildGraphNode(&node, c->graph, &c->root, 1, ch->graph));
  return IEX_OK;
}

// A new constructor whose graph runs all the given graphs side by side under one root.
extern "C" void* iex_graph_combine(void* const* handles, int count) {
  if (count < 0 || (count > 0 && !handles)) return nullptr;
  void* h = iex_graph_create();
  if (!h) return nullptr;
  for (int i = 0; i < count; ++i)
    if (iex_graph_add_child(h, handles[i]) != IEX_OK) {
      iex_graph_destroy(h);
      return nullptr;
    }
  return h;
}
