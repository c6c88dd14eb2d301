// Expert parallelism across the GPUs of one node: experts are split into
// contiguous ranges, attention / dense weights / router / KV are replicated, so
// every GPU already holds the hidden state and the routing decision and
// "dispatch" moves no data.  The only exchange is one sum of the [T, hidden]
// partial MoE outputs per layer (NCCL all-reduce over NVLink).  The reference's
// nearest analogue is NUMA-sticky expert placement with per-node pools
// (core/src/llm/moe/native.cpp:1196,1506-1567).
//
// NCCL is loaded at run time (dlopen) so single-GPU use has no dependency on it.
#include <dlfcn.h>
#include <string.h>

#include "dc_internal.h"
#include "dc_model.h"

typedef struct ncclComm* ncclComm_t;
typedef struct { char internal[128]; } ncclUniqueId;
typedef int ncclResult_t;
enum { ncclFloat32 = 7, ncclSum = 0 };

struct NcclApi {
    ncclResult_t (*GetUniqueId)(ncclUniqueId*);
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int);
    ncclResult_t (*AllReduce)(const void*, void*, size_t, int, int, ncclComm_t, cudaStream_t);
    ncclResult_t (*CommDestroy)(ncclComm_t);
    const char* (*GetErrorString)(ncclResult_t);
};
static NcclApi g_nccl;
static void* g_nccl_lib = nullptr;

static int load_nccl(dc_ctx* ctx, const char* path) {
    if (g_nccl_lib) return DC_B200_OK;
    const char* cands[] = {path, "libnccl.so.2", "libnccl.so"};
    for (const char* c : cands) {
        if (!c || !*c) continue;
        g_nccl_lib = dlopen(c, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl_lib) break;
    }
    if (!g_nccl_lib) return dc_fail(ctx, DC_B200_BACKEND_ERROR, "cannot load NCCL: %s", dlerror());
    g_nccl.GetUniqueId = (decltype(g_nccl.GetUniqueId))dlsym(g_nccl_lib, "ncclGetUniqueId");
    g_nccl.CommInitRank = (decltype(g_nccl.CommInitRank))dlsym(g_nccl_lib, "ncclCommInitRank");
    g_nccl.AllReduce = (decltype(g_nccl.AllReduce))dlsym(g_nccl_lib, "ncclAllReduce");
    g_nccl.CommDestroy = (decltype(g_nccl.CommDestroy))dlsym(g_nccl_lib, "ncclCommDestroy");
    g_nccl.GetErrorString = (decltype(g_nccl.GetErrorString))dlsym(g_nccl_lib, "ncclGetErrorString");
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.CommDestroy)
        return dc_fail(ctx, DC_B200_BACKEND_ERROR, "NCCL library lacks a required symbol");
    return DC_B200_OK;
}

int dc_ep_allreduce(dc_model* m, float* buf, size_t n) {
    if (!m->ep_ready) return dc_fail(m->ctx, DC_B200_BACKEND_ERROR, "expert-parallel communicator not initialised");
    ncclResult_t r = g_nccl.AllReduce(buf, buf, n, ncclFloat32, ncclSum, (ncclComm_t)m->ep_comm, m->ctx->stream);
    if (r != 0) return dc_fail(m->ctx, DC_B200_BACKEND_ERROR, "ncclAllReduce: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error");
    return DC_B200_OK;
}

void dc_ep_destroy(dc_model* m) {
    if (m->ep_comm && g_nccl.CommDestroy) g_nccl.CommDestroy((ncclComm_t)m->ep_comm);
    m->ep_comm = nullptr;
    m->ep_ready = false;
}

extern "C" {

// 128-byte id created on rank 0 and handed to every rank by the launcher
// (torch.distributed broadcast in the benchmark).
int dc_b200_ep_unique_id(dc_ctx* ctx, const char* nccl_path, void* id_out_128) {
    if (!ctx || !id_out_128) return DC_B200_INVALID_ARGUMENT;
    int st = load_nccl(ctx, nccl_path);
    if (st != DC_B200_OK) return st;
    ncclUniqueId id;
    ncclResult_t r = g_nccl.GetUniqueId(&id);
    if (r != 0) return dc_fail(ctx, DC_B200_BACKEND_ERROR, "ncclGetUniqueId failed (%d)", r);
    memcpy(id_out_128, &id, 128);
    return DC_B200_OK;
}

int dc_b200_model_ep_init(dc_model* m, const char* nccl_path, const void* id_128) {
    if (!m || !id_128) return DC_B200_INVALID_ARGUMENT;
    if (m->cfg.ep_size <= 1) return DC_B200_OK;
    int st = load_nccl(m->ctx, nccl_path);
    if (st != DC_B200_OK) return st;
    cudaSetDevice(m->ctx->device);
    ncclUniqueId id;
    memcpy(&id, id_128, 128);
    ncclComm_t comm = nullptr;
    ncclResult_t r = g_nccl.CommInitRank(&comm, m->cfg.ep_size, id, m->cfg.ep_rank);
    if (r != 0) return dc_fail(m->ctx, DC_B200_BACKEND_ERROR, "ncclCommInitRank: %s", g_nccl.GetErrorString ? g_nccl.GetErrorString(r) : "error");
    m->ep_comm = comm;
    m->ep_ready = true;
    return DC_B200_OK;
}

}  // extern "C"
