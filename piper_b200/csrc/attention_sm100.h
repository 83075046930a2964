// Host-side launchers of the causal GQA flash-attention kernels
// (attention_sm100.cu).  qkv is the packed bf16 projection
// [B*S, (Hq + 2*Hkv) * hd] with rotary embedding already applied; S must be
// a multiple of 128 and hd 64 or 128.  Return codes: 0 ok, -1 unsupported
// shape, -2 kernel attribute set-up failed, -3 launch error, >0 CUresult of
// a tensor-map encode.
#pragma once
#include <cuda_runtime.h>

namespace piper {

// out [B*S, Hq*hd] bf16, lse [B, Hq, S] fp32 (natural log).
int attn_fwd(const void* qkv, void* out, float* lse, int B, int S, int Hq, int Hkv, int hd,
             float softmax_scale, int* status, cudaStream_t st);

// d_qkv has the layout of qkv and is fully overwritten.  delta is scratch of
// B*Hq*S floats provided by the caller.
int attn_bwd(const void* qkv, const void* out, const void* d_out, const float* lse, float* delta,
             void* d_qkv, int B, int S, int Hq, int Hkv, int hd, float softmax_scale, int* status,
             cudaStream_t st);

}  // namespace piper
