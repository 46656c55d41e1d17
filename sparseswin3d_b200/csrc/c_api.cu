// Status strings and the last-CUDA-error record of the C ABI.
#include <stdio.h>
#include <string.h>

#include "ssw_common.cuh"

namespace ssw {
static thread_local char g_cuda_error[256] = "";
void set_cuda_error(cudaError_t e, const char* where) {
  snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}
void set_error_text(const char* text) { snprintf(g_cuda_error, sizeof(g_cuda_error), "%s", text); }
}  // namespace ssw

extern "C" const char* ssw_status_string(int status) {
  switch (status) {
    case SSW_OK: return "ok";
    case SSW_E_INVALID: return "invalid argument";
    case SSW_E_RANGE: return "size outside the int32 domain of the layout";
    case SSW_E_UNSUPPORTED: return "configuration outside the compiled variants";
    case SSW_E_CUDA: return "CUDA runtime error";
    case SSW_E_WORKSPACE: return "workspace too small";
    default: return "unknown status";
  }
}

extern "C" const char* ssw_last_cuda_error(void) { return ssw::g_cuda_error; }

extern "C" int ssw_version(void) { return 200; }

extern "C" int ssw_enable_peer_access(int32_t peer_device) {
  int dev = 0, can = 0;
  SSW_CUDA_TRY(cudaGetDevice(&dev));
  if (peer_device == dev) return SSW_OK;
  SSW_CUDA_TRY(cudaDeviceCanAccessPeer(&can, dev, peer_device));
  if (!can) return SSW_E_UNSUPPORTED;
  const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
  if (e == cudaErrorPeerAccessAlreadyEnabled) {
    (void)cudaGetLastError();  // clear the sticky-free error state
    return SSW_OK;
  }
  if (e != cudaSuccess) {
    ssw::set_cuda_error(e, "cudaDeviceEnablePeerAccess");
    return SSW_E_CUDA;
  }
  return SSW_OK;
}

static_assert(sizeof(cudaIpcMemHandle_t) == SSW_IPC_HANDLE_BYTES, "IPC handle size");

extern "C" int ssw_peer_buffer_create(int64_t bytes, void** ptr, unsigned char* handle) {
  if (bytes <= 0 || !ptr || !handle) return SSW_E_INVALID;
  void* p = nullptr;
  SSW_CUDA_TRY(cudaMalloc(&p, (size_t)bytes));
  cudaIpcMemHandle_t h;
  cudaError_t e = cudaMemset(p, 0, (size_t)bytes);
  if (e == cudaSuccess) e = cudaDeviceSynchronize();
  if (e == cudaSuccess) e = cudaIpcGetMemHandle(&h, p);
  if (e != cudaSuccess) {
    (void)cudaFree(p);
    ssw::set_cuda_error(e, "ssw_peer_buffer_create");
    return SSW_E_CUDA;
  }
  memcpy(handle, &h, sizeof(h));
  *ptr = p;
  return SSW_OK;
}

extern "C" int ssw_peer_buffer_open(const unsigned char* handle, void** ptr) {
  if (!handle || !ptr) return SSW_E_INVALID;
  cudaIpcMemHandle_t h;
  memcpy(&h, handle, sizeof(h));
  // opened in the context of the current device: that is the device whose kernels will use *ptr
  SSW_CUDA_TRY(cudaIpcOpenMemHandle(ptr, h, cudaIpcMemLazyEnablePeerAccess));
  return SSW_OK;
}

extern "C" int ssw_peer_buffer_close(void* ptr) {
  if (!ptr) return SSW_E_INVALID;
  SSW_CUDA_TRY(cudaIpcCloseMemHandle(ptr));
  return SSW_OK;
}

extern "C" int ssw_peer_buffer_destroy(void* ptr) {
  if (!ptr) return SSW_E_INVALID;
  SSW_CUDA_TRY(cudaFree(ptr));
  return SSW_OK;
}

// Host-side debug helper: the dependency edges of a captured CUDA graph as text, one edge per line,
//   <from> -> <to> <full|programmatic> from_port=<p> to_port=<p>
// with nodes written as <index>:<name>, kernel nodes named by their function and other nodes by
// their type number.  Lets a caller
// check how a captured sequence of this library's chained launches was wired (which edges became
// programmatic, and that a cross-stream join is a full dependency).  Touches no device memory.
static void node_name(cudaGraphNode_t n, char* out, size_t cap) {
  cudaGraphNodeType t;
  if (cudaGraphNodeGetType(n, &t) != cudaSuccess) {
    snprintf(out, cap, "?");
    return;
  }
  if (t == cudaGraphNodeTypeKernel) {
    cudaKernelNodeParams kp;
    const char* name = nullptr;
    if (cudaGraphKernelNodeGetParams(n, &kp) == cudaSuccess && kp.func && cudaFuncGetName(&name, kp.func) == cudaSuccess &&
        name) {
      snprintf(out, cap, "%s", name);
      return;
    }
    // a kernel the runtime cannot describe (a library's, loaded through the driver API): the failed
    // query must not stay behind as the thread's last error
    (void)cudaGetLastError();
    snprintf(out, cap, "kernel");
    return;
  }
  snprintf(out, cap, "node_type_%d", (int)t);
}

extern "C" int ssw_debug_graph_edges(void* graph_, char* text, int64_t text_bytes, int64_t* n_nodes, int64_t* n_edges,
                                     int64_t* n_programmatic) {
  cudaGraph_t graph = (cudaGraph_t)graph_;
  if (!graph || !text || text_bytes < 1) return SSW_E_INVALID;
  size_t nn = 0, ne = 0;
  SSW_CUDA_TRY(cudaGraphGetNodes(graph, nullptr, &nn));
  SSW_CUDA_TRY(cudaGraphGetEdges_v2(graph, nullptr, nullptr, nullptr, &ne));
  cudaGraphNode_t* nodes = new cudaGraphNode_t[nn + 1];
  if (nn > 0 && cudaGraphGetNodes(graph, nodes, &nn) != cudaSuccess) nn = 0;
  auto index_of = [&](cudaGraphNode_t n) {
    for (size_t i = 0; i < nn; ++i)
      if (nodes[i] == n) return (int)i;
    return -1;
  };
  cudaGraphNode_t* from = new cudaGraphNode_t[ne + 1];
  cudaGraphNode_t* to = new cudaGraphNode_t[ne + 1];
  cudaGraphEdgeData* ed = new cudaGraphEdgeData[ne + 1];
  int status = SSW_OK;
  int64_t prog = 0, pos = 0;
  text[0] = 0;
  if (ne > 0 && cudaGraphGetEdges_v2(graph, from, to, ed, &ne) != cudaSuccess) {
    ssw::set_cuda_error(cudaGetLastError(), "cudaGraphGetEdges_v2");
    status = SSW_E_CUDA;
  } else {
    for (size_t i = 0; i < ne; ++i) {
      char a[200], b[200];
      node_name(from[i], a, sizeof(a));
      node_name(to[i], b, sizeof(b));
      const bool p = ed[i].type == cudaGraphDependencyTypeProgrammatic;
      prog += p;
      const int w = snprintf(text + pos, (size_t)(text_bytes - pos), "%d:%s -> %d:%s %s from_port=%d to_port=%d\n",
                             index_of(from[i]), a, index_of(to[i]), b, p ? "programmatic" : "full", (int)ed[i].from_port,
                             (int)ed[i].to_port);
      if (w < 0 || pos + w >= text_bytes) {
        status = SSW_E_WORKSPACE;
        break;
      }
      pos += w;
    }
  }
  delete[] nodes;
  delete[] from;
  delete[] to;
  delete[] ed;
  (void)cudaGetLastError();  // a read-only helper leaves no error state behind
  if (n_nodes) *n_nodes = (int64_t)nn;
  if (n_edges) *n_edges = (int64_t)ne;
  if (n_programmatic) *n_programmatic = prog;
  return status;
}
