// Split-KV attention for a few query rows per key/value head (fmha_decode.cu).
#pragma once
#include "common.cuh"
#include "host.h"

namespace b200k {

constexpr int kFmhaDecodeMaxRows = 8;   // seq_q * query_group_size handled by the decode kernels

bool fmha_decode_applies(const b200k_fmha_args* a);
int64_t fmha_decode_workspace_bytes(const b200k_fmha_args* a, int sms);
// `a->workspace` must hold fmha_decode_workspace_bytes(a, sms) bytes.
int launch_fmha_decode(const b200k_fmha_args* a, int sms, cudaStream_t stream);

}  // namespace b200k
