// seq_engine.h -- the layered sequence engine: models described by a LIST of layers in config.json (each with a mixer of some type
// and an optional feed-forward), served by one ragged step function over a paged KV pool and a pool of state slots.
//
// It is the second model executor of the library beside TextModel (the fixed Qwen3 stack): the same handle, weight table, paged
// cache idea (32-token pages handed out from one free list), sampler kernels and batch-session entry points, but
//   * a step takes ANY mix of entries -- a portion of a prompt for one sequence beside single decoded tokens of others;
//   * a sequence owns a state slot (recurrent state, convolution tails, sampler state) next to its pages;
//   * layers are built from the mixer / feed-forward registry in seq_engine.cu, so another layer list needs no new code.
// This header is all api.cu sees; the kernels live in seq_engine.cu's translation unit.
#pragma once
#include <cstddef>
#include <cstdint>
#include <string>
#include <vector>

#include "../../include/aha_b200.h"

namespace aha {

struct Ctx;
struct Json;
struct WeightTable;

struct SeqStepEntry {
    int slot = -1;
    const uint32_t* tokens = nullptr;   // n ids, or nullptr with n == 1: the token the slot's sampler produced last (it never left the device)
    int n = 0;
    const int32_t* want = nullptr;      // indices into this entry's tokens whose logits are wanted, ascending
    int n_want = 0;
    bool sample = false;                // run the slot's sampler on the logits of the entry's LAST token (which need not be in `want`)
};

struct SeqEngineOptions {
    int max_tokens = 8192;        // KV capacity of the pool, in tokens (rounded up to pages)
    int max_seqs = 8;             // state slots
    int max_step_tokens = 2048;   // tokens one launch sequence carries; longer steps are cut into portions by the scheduler
    bool fp32 = false;            // true: weights widened to fp32 and every product in fp32; false: bf16 weights, bf16 tensor-core products where they apply
    bool use_graph = true;        // replay decode-only steps from CUDA graphs
    int gemm_impl = 0;            // 0 = auto, 1 = CUDA-core kernels only
    int seq_impl = 0;             // sequence kernels (attention, recurrence): 0 = auto (the fast ones where the sizes allow), 1 = the plain ones only
};

class SeqEngine {
  public:
    virtual ~SeqEngine() {}
    virtual int vocab() const = 0;
    virtual int max_seqs() const = 0;
    virtual int page_tokens() const = 0;
    virtual size_t free_tokens() const = 0;             // unmapped KV capacity
    virtual int admit() = 0;                            // a free slot, positioned at 0; throws when none is free
    virtual void release(int slot) = 0;                 // pages back to the free list, slot free
    virtual void release_all() = 0;
    virtual bool live(int slot) const = 0;
    virtual int position(int slot) const = 0;           // tokens the sequence holds
    virtual void set_sampler(int slot, const aha_gen_params& p) = 0;   // also clears the slot's history and draw counter
    // One engine step.  logits_out (host, may be nullptr): rows of all `want` indices in entry order, [rows][vocab].
    // tokens_out (host, may be nullptr): [n] the sampled token of every entry with sample == true.
    virtual void step(const SeqStepEntry* entries, int n, float* logits_out, uint32_t* tokens_out) = 0;
    // residual stream after every layer of the LAST launch sequence ([layers][T][width]); tracing must have been switched on before the step
    virtual void set_trace(bool on) = 0;
    virtual size_t read_trace(int layer, float* out, size_t cap) = 0;
    virtual uint64_t weight_bytes() const = 0;
    virtual uint64_t kv_bytes_per_token() const = 0;
    // Device-timed steps on synthetic tokens (n_seqs sequences x tokens_per_seq tokens at context ctx) -> JSON: ms per step (CUDA events around
    // `iters` whole steps, scheduler and host copies included) and, from separate runs with events around every launch family, the time,
    // algorithmic FLOPs and bytes of each family summed over the layers.  Frees every slot.
    virtual std::string profile(int n_seqs, int tokens_per_seq, int ctx, int warmup, int iters) = 0;
};

// config: the checkpoint's config.json (a "layers" list); throws on anything it does not know
SeqEngine* make_layered_engine(Ctx& ctx, const Json& config, const WeightTable& wt, const SeqEngineOptions& opt);

}  // namespace aha
