// Kernel launch helper: every kernel of a decoder step is launched with the
// programmatic-stream-serialization attribute so that its prologue (weight
// prefetch) overlaps the tail of the previous kernel.
#pragma once
#include "dc_internal.h"

template <typename... KArgs, typename... Args>
static inline int dc_launch(dc_ctx* ctx, const char* name, void (*kernel)(KArgs...), dim3 grid, dim3 block,
                            size_t smem, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ctx->use_pdl ? 1 : 0;
    return dc_check_cuda(ctx, cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...), name);
}
