// dflash_verify_step: one speculative-verify step over a hybrid stack in a handful of launches.
//
// The reference's cycle (Sources/DFlash/DFlashRuntime.swift:499-579) runs one kernel per gated-delta layer
// for the verify forward and again for the rollback, and reads the accepted length on the host in between
// (:525-530).  Here the layers of a kind are folded into the batch axis of one launch each and the accepted
// length never leaves the device: forward over B * gdn_layers items, attention over B * attn_layers
// sequences, posterior + acceptance, then the delta-tape replay and the conv windows over B * gdn_layers
// items, every item of a sequence reading that sequence's replay length.
#include "common.cuh"

namespace dflash {
namespace {

int32_t bad_desc(const char* what) {
  set_error("verify_step: %s", what);
  return DFLASH_ERR_INVALID_ARG;
}

}  // namespace
}  // namespace dflash

using namespace dflash;

extern "C" size_t dflash_verify_step_workspace_bytes(const dflash_verify_step_desc* d) {
  if (!d || d->attn_layers <= 0) return 0;
  if (d->kv_format == DFLASH_KV_TURBO3 && d->attn_k) {
    const dflash_turbo_kv* t = reinterpret_cast<const dflash_turbo_kv*>(d->attn_k);
    return dflash_verify_sdpa_turbo_workspace_bytes(d->B * d->attn_layers, d->Hq, d->Hkv, d->D, t->n_cold, t->n_hot);
  }
  return dflash_verify_sdpa_workspace_bytes_ex(d->B * d->attn_layers, d->Hq, d->Hkv, d->D, d->N, d->kv_format);
}

extern "C" int32_t dflash_verify_step(const dflash_verify_step_desc* d, void* workspace, size_t workspace_bytes,
                                      void* stream) {
  if (!d) return bad_desc("null descriptor");
  if (d->B <= 0 || d->T <= 0) return bad_desc("non-positive batch or block length");
  if (!d->logits || !d->verify_ids || !d->posterior || !d->accept || !d->replay_len) return bad_desc("null acceptance array");
  if ((long long)d->B * (d->gdn_layers > d->attn_layers ? d->gdn_layers : d->attn_layers) > 0x7fffffffLL / 64) return bad_desc("too many items");
  cudaStream_t s = reinterpret_cast<cudaStream_t>(stream);
  const int items = d->B * d->gdn_layers;

  // 1. verify forward of every gated-delta layer over the whole block, tape recorded
  if (d->gdn_layers > 0) {
    if (!d->tape || !d->state_rolled) return bad_desc("null gated-delta output");
    if (d->state_verify) {
      if (int32_t st = dflash_gated_delta_tape(d->q, d->k, d->v, d->g, d->beta, d->state, nullptr, nullptr, d->y, d->state_verify,
                                               d->tape, items, d->T, d->Hk, d->Hv, d->Dk, d->Dv, d->g_is_vector, d->in_dtype, 0, stream))
        return st;
    } else {
      // The state after all T steps is not wanted: every sequence's result state is the rollback's (state_rolled; for a
      // fully accepted block the two are the same state).  The tensor-core kernel then writes no state at all.
      if (!d->q || !d->k || !d->v || !d->g || !d->beta || !d->state || !d->y) return bad_desc("null gated-delta input");
      GdnArgs a{d->q, d->k, d->v, d->g, d->beta, d->state, nullptr, nullptr, d->y, nullptr, d->tape,
                items, d->T, d->Hk, d->Hv, d->Dk, d->Dv, d->g_is_vector ? 1 : 0, d->in_dtype, 0, false};
      if (!gdn_tc_supported(a)) return bad_desc("state_verify may be NULL only for bf16 inputs, Dk = Dv = 128, a scalar gate and T <= 16");
      if (int32_t st = launch_gdn_tc(a, s)) return st;
    }
  }
  // 2. block-verify attention of every attention layer
  if (d->attn_layers > 0) {
    if (int32_t st = dflash_verify_sdpa(d->attn_q, d->attn_k, d->attn_v, nullptr, nullptr, nullptr, d->attn_out, workspace,
                                        workspace_bytes, d->B * d->attn_layers, d->Hq, d->Hkv, d->T, d->D, d->N, 0, 0, 0, d->scale,
                                        d->attn_dtype, d->kv_format, stream))
      return st;
  }
  // 3. greedy posterior, accepted length, next token, replay length (DFlashRuntime.swift:513-547)
  if (int32_t st = dflash_greedy_tokens(d->logits, d->suppress, d->posterior, d->B * d->T, d->V, d->logits_dtype, stream)) return st;
  if (int32_t st = dflash_accept_lengths(d->posterior, d->verify_ids, d->accept, d->next_token, d->replay_len, d->B, d->T, stream)) return st;
  if (d->logits_rows)
    if (int32_t st = dflash_gather_logits_rows(d->logits, d->accept, d->logits_rows, d->B, d->T, d->V, d->logits_dtype, stream)) return st;
  // 4. rollback of every gated-delta layer to its sequence's replay length (RecurrentRollbackCache.swift:115-127)
  if (d->gdn_layers > 0) {
    GdnArgs a{nullptr, d->k, nullptr, d->g, nullptr, d->state, nullptr, d->replay_len, nullptr, d->state_rolled, d->tape,
              items, d->T, d->Hk, d->Hv, d->Dk, d->Dv, d->g_is_vector ? 1 : 0, d->in_dtype, 0, true, d->gdn_layers};
    if (int32_t st = gdn_fast_supported(a) ? launch_gdn_fast(a, s) : launch_gdn_generic(a, s)) return st;
    if (d->qkv && d->conv_out) {
      if (d->conv_keep <= 0 || d->conv_row_bytes <= 0 || d->conv_row_bytes % 16 != 0) return bad_desc("conv window rows must be multiples of 16 bytes");
      if (int32_t st = launch_conv_window(d->conv_snapshot, d->qkv, d->replay_len, 0, d->conv_out, items, d->T, d->conv_keep,
                                          d->conv_row_bytes, nullptr, d->gdn_layers, s))
        return st;
    }
  }
  return DFLASH_OK;
}
