// Per-request state that lives on the device, and the two small kernels that open and close a step.
//
// The reference keeps what it knows about a request on the host (RequestInfo: block ids and sequence length,
// src/model/kv_manager.py:9-16) and rebuilds a device copy of the block tables and context lengths for every
// decode step (build_decode_metadata, src/model/kv_manager.py:521-561). Here that state is a fixed-size record
// per request SLOT in one int32 array on the device, the "slot store":
//
//   len[slot]    tokens of the request that are in the cache (= position of its next token)
//   last[slot]   the token sampled for it last (the next input of a decode step that feeds tokens back)
//   temp[slot]   sampling temperature (float bits)        seed[slot]   sampling seed (64 bit)
//   table g      block table of cache group g, [slots + 1][width_g] page ids, -1 = no page
//
// The host uploads, per step, only what the device cannot know: which slots take part (item_slot), how the
// step's tokens are cut into items (q_start), the wanted rows, the token ids unless the device fed them back,
// and a list of (offset, value) corrections of the store: the page ids that the step's new positions needed,
// sampling parameters of newly admitted requests, a length where the host's bookkeeping and the device's
// differ (a new request in a used slot, a step that was launched ahead and then dropped).
//
// step_begin applies the corrections, then expands the slots' state into the per-step arrays that every other
// kernel reads (positions, token -> item, token -> block-table row, length after the step, sampling
// parameters) and moves each slot's length on by the step's tokens. step_end (after sampling) stores the
// sampled tokens in the slots and in the host-visible history of the run.
#include "common.cuh"

namespace ps {

struct SlotStoreView {
    int* base;          // the store
    int size;           // words
    int len, last, temp, seed;   // offsets of the sections (seed: two words per slot)
    int slots;          // request slots; slot index `slots` is the scratch slot of padding entries
};

struct StepLayoutView {
    int* meta;          // the step's packed metadata
    int T, I;           // tokens, items
    // uploaded by the host
    int header;         // [0] steps run since the upload, [1] tokens fed back on the device, [2] corrections
    int item_slot, q_start, updates, update_capacity, token_ids;
    // written here
    int positions, token_item, token_slot, kv_len, temperature, seed;
};

constexpr int BEGIN_THREADS = 1024;

// One CTA: the three phases depend on one another and a step has at most a few thousand tokens.
__global__ void __launch_bounds__(BEGIN_THREADS)
step_begin_kernel(SlotStoreView store, StepLayoutView step, int* __restrict__ status) {
    pdl_prologue();                                   // the step before may still be writing last[] and the header
    int* meta = pdl_fresh(step.meta);
    int* base = pdl_fresh(store.base);
    const int tid = threadIdx.x;
    const int* header = meta + step.header;
    const int fed = header[1];
    int n_updates = header[2];
    bool bad = false;
    if (n_updates < 0 || n_updates > step.update_capacity) {
        bad = true;
        n_updates = 0;
    }
    // 1. corrections of the store
    const int* updates = meta + step.updates;
    for (int u = tid; u < n_updates; u += BEGIN_THREADS) {
        const int offset = updates[2 * u], value = updates[2 * u + 1];
        if (offset < 0 || offset >= store.size) bad = true;
        else base[offset] = value;
    }
    __syncthreads();
    // 2. per item: where the request stands, where it will stand, how it samples
    const int* item_slot = meta + step.item_slot;
    const int* q_start = meta + step.q_start;
    for (int i = tid; i < step.I; i += BEGIN_THREADS) {
        const int slot = item_slot[i];
        const int first = q_start[i], count = q_start[i + 1] - first;
        if (slot < 0 || slot > store.slots || count < 0) {
            bad = true;
            meta[step.kv_len + i] = 0;
            continue;
        }
        int start = 0;
        if (slot < store.slots) {                     // the scratch slot always starts at 0 and may come twice
            start = base[store.len + slot];
            base[store.len + slot] = start + count;
        }
        meta[step.kv_len + i] = start + count;
        meta[step.temperature + i] = base[store.temp + slot];
        meta[step.seed + 2 * i] = base[store.seed + 2 * slot];
        meta[step.seed + 2 * i + 1] = base[store.seed + 2 * slot + 1];
        if (fed && count == 1) meta[step.token_ids + first] = base[store.last + slot];
    }
    __syncthreads();
    // 3. per token: its item (the last one that starts at or before it and is not empty), position and table row
    for (int t = tid; t < step.T; t += BEGIN_THREADS) {
        int lo = 0, hi = step.I;                      // invariant: q_start[lo] <= t < q_start[hi]
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if (q_start[mid] <= t) lo = mid; else hi = mid;
        }
        const int count = q_start[lo + 1] - q_start[lo];
        const int slot = item_slot[lo];
        meta[step.token_item + t] = lo;
        meta[step.token_slot + t] = (slot < 0 || slot > store.slots) ? store.slots : slot;
        meta[step.positions + t] = meta[step.kv_len + lo] - count + (t - q_start[lo]);
    }
    if (bad && status) atomicExch(status, 4);
}

// After a step that sampled on the device: the sampled token of item i becomes last[slot] (the next step's
// input if it feeds back) and is appended to the history of the run, which may be host memory mapped for the
// device; the header then says that one more step has run and that tokens are fed back, with no corrections
// pending. status (may be null) is copied to *status_copy for the host to read along with the tokens.
__global__ void step_end_kernel(SlotStoreView store, StepLayoutView step, const int* __restrict__ sampled,
                                int* __restrict__ history, int B, int max_steps, const int* status,
                                int* status_copy) {
    pdl_prologue();
    sampled = pdl_fresh(sampled);
    int* meta = pdl_fresh(step.meta);
    int* header = meta + step.header;
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    const int run = header[0];
    // every kernel of the step has ended: what they flagged travels with the tokens
    const int flagged = (i == 0 && status && status_copy) ? *(volatile const int*)status : 0;
    if (i < B) {
        const int token = sampled[i];
        const int slot = meta[step.item_slot + i];
        if (slot >= 0 && slot < store.slots) store.base[store.last + slot] = token;
        if (run < max_steps) history[(size_t)run * B + i] = token;
    }
    __syncthreads();
    if (i == 0) {
        header[0] = run + 1;
        header[1] = 1;
        header[2] = 0;
        if (flagged) *status_copy = flagged;              // the host zeroed the copy and zeroes it after a read
    }
}

}  // namespace ps

// store_layout: {size, len, last, temp, seed, slots}; step_layout: {T, I, header, item_slot, q_start, updates,
// update_capacity, token_ids, positions, token_item, token_slot, kv_len, temperature, seed} (word offsets).
static bool make_views(int* store, const int* store_layout, int* meta, const int* step_layout,
                       ps::SlotStoreView* sv, ps::StepLayoutView* lv) {
    if (!store || !store_layout || !meta || !step_layout) return false;
    *sv = ps::SlotStoreView{store, store_layout[0], store_layout[1], store_layout[2], store_layout[3],
                            store_layout[4], store_layout[5]};
    *lv = ps::StepLayoutView{meta, step_layout[0], step_layout[1], step_layout[2], step_layout[3], step_layout[4],
                             step_layout[5], step_layout[6], step_layout[7], step_layout[8], step_layout[9],
                             step_layout[10], step_layout[11], step_layout[12], step_layout[13]};
    return sv->size > 0 && sv->slots > 0 && lv->T > 0 && lv->I > 0 && lv->update_capacity >= 0;
}

PS_EXPORT int ps_step_begin(int* store, const int* store_layout, int* meta, const int* step_layout, int* status,
                            void* stream) {
    ps::SlotStoreView sv;
    ps::StepLayoutView lv;
    if (!make_views(store, store_layout, meta, step_layout, &sv, &lv)) return PS_ERR_BAD_ARGUMENT;
    return ps::launch_pdl(ps::step_begin_kernel, dim3(1), dim3(ps::BEGIN_THREADS), 0, (cudaStream_t)stream, sv, lv,
                          status);
}

// One block: B <= 1024 items of one token each.
PS_EXPORT int ps_step_end(int* store, const int* store_layout, int* meta, const int* step_layout,
                          const int* sampled, int* history, int B, int max_steps, const int* status,
                          int* status_copy, void* stream) {
    ps::SlotStoreView sv;
    ps::StepLayoutView lv;
    if (!make_views(store, store_layout, meta, step_layout, &sv, &lv)) return PS_ERR_BAD_ARGUMENT;
    if (B <= 0) return PS_OK;
    if (B > 1024 || B != lv.I || !sampled || !history) return PS_ERR_UNSUPPORTED;
    return ps::launch_pdl(ps::step_end_kernel, dim3(1), dim3(((B + 31) / 32) * 32), 0, (cudaStream_t)stream, sv, lv,
                          sampled, history, B, max_steps, status, status_copy);
}
