// Host side of a step, natively: lay the entries of a step out as one flat batch and write what the host
// uploads into the step's staging buffer.
//
// The reference builds its flat batch in Python lists and tensors per step (build_iteration_batch,
// src/scheduler/orca_scheduler.py:171-219). Here the arrangement is specified by the pure function
// `arrange_step` of pagedserve_b200/engine/batch.py (short entries first, prompt portions after them, optional
// padding to recurring shapes); the two functions below compute the same thing without the interpreter: a few
// dozen small numpy calls cost about 100 us per step, this costs a few. Host code only: no kernel here.
#include "common.cuh"

namespace {

inline long long round_up(long long v, long long step) { return (v + step - 1) / step * step; }

struct Shape {
    int T, I, R, num_short_items, num_short_tokens, num_long_blocks, real_rows, max_q_len, max_kv_len;
    // what the fill needs besides
    int real_short, real_long, extra_short, extra_long, short_items, long_items;
};

// counts / starts / want_counts are per entry, in the caller's order.
bool shape_of(int n, const long long* counts, const long long* starts, const int* want_counts, int long_entry,
              int pad, int pad_short, int pad_long, Shape* s) {
    long long short_tokens = 0, long_tokens = 0, long_blocks = 0, max_q = 0, max_kv = 0;
    int num_short = 0, num_long = 0, rows = 0;
    for (int i = 0; i < n; ++i) {
        const long long c = counts[i];
        if (c <= 0) return false;
        if (c < long_entry) { ++num_short; short_tokens += c; }
        else { ++num_long; long_tokens += c; long_blocks += (c + 63) / 64; }
        if (c > max_q) max_q = c;
        if (starts[i] + c > max_kv) max_kv = starts[i] + c;
        rows += want_counts[i];
    }
    s->real_short = num_short;
    s->real_long = num_long;
    s->real_rows = rows;
    s->extra_short = s->extra_long = 0;
    s->short_items = num_short;
    s->long_items = num_long;
    s->R = rows;
    if (pad) {
        s->extra_short = (int)(round_up(short_tokens, pad_short) - short_tokens);
        s->extra_long = (int)(round_up(long_tokens, pad_long) - long_tokens);
        s->short_items = short_tokens ? (int)round_up(num_short + (s->extra_short > 0), 8) : 0;
        s->long_items = long_tokens ? (int)round_up(num_long + (s->extra_long > 0), 4) : 0;
        s->R = (int)round_up(rows, 8);
        // a bound that depends on the padded shape alone
        long_blocks = (long_tokens + s->extra_long) / 64 + s->long_items;
        if (s->extra_short > max_q) max_q = s->extra_short;
        if (s->extra_long > max_q) max_q = s->extra_long;
        if (s->extra_short > max_kv) max_kv = s->extra_short;
        if (s->extra_long > max_kv) max_kv = s->extra_long;
    }
    s->T = (int)(short_tokens + long_tokens + s->extra_short + s->extra_long);
    s->I = s->short_items + s->long_items;
    s->num_short_items = s->short_items;
    s->num_short_tokens = (int)(short_tokens + s->extra_short);
    s->num_long_blocks = (int)long_blocks;
    s->max_q_len = (int)max_q;
    s->max_kv_len = (int)max_kv;
    return true;
}

}  // namespace

// shape_out[9] = {T, I, R, num_short_items, num_short_tokens, num_long_blocks, real_rows, max_q_len, max_kv_len}
PS_EXPORT int ps_step_shape(int n, const long long* counts, const long long* starts, const int* want_counts,
                            int long_entry, int pad, int pad_short, int pad_long, int* shape_out) {
    if (n <= 0 || !counts || !starts || !want_counts || !shape_out) return PS_ERR_BAD_ARGUMENT;
    Shape s;
    if (!shape_of(n, counts, starts, want_counts, long_entry, pad, pad_short, pad_long, &s)) return PS_ERR_BAD_ARGUMENT;
    const int values[9] = {s.T, s.I, s.R, s.num_short_items, s.num_short_tokens, s.num_long_blocks, s.real_rows,
                           s.max_q_len, s.max_kv_len};
    memcpy(shape_out, values, sizeof(values));
    return PS_OK;
}

// Writes item_slot[I], q_start[I + 1], logit_rows[R] and token_ids[T] (int32) at the given word offsets of
// `staging`. tokens: all token ids in the caller's order, entry after entry (int64). slots: per entry.
// wants: the wanted places of all entries, entry after entry. vocab: token ids must lie in [0, vocab).
// Returns PS_ERR_BAD_ARGUMENT for a token outside the vocabulary (bad_token receives it).
PS_EXPORT int ps_step_fill(int n, const long long* counts, const long long* starts, const int* want_counts,
                           const long long* tokens, const long long* slots, const int* wants, int long_entry,
                           int pad, int pad_short, int pad_long, int scratch_slot, long long vocab, int* staging,
                           int off_item_slot, int off_q_start, int off_logit_rows, int off_token_ids,
                           long long* bad_token) {
    if (n <= 0 || !staging || !tokens || !slots) return PS_ERR_BAD_ARGUMENT;
    Shape s;
    if (!shape_of(n, counts, starts, want_counts, long_entry, pad, pad_short, pad_long, &s)) return PS_ERR_BAD_ARGUMENT;
    int* item_slot = staging + off_item_slot;
    int* q_start = staging + off_q_start;
    int* logit_rows = staging + off_logit_rows;
    int* token_ids = staging + off_token_ids;
    // first token of every entry in the caller's order (for the wanted rows), filled while laying out
    int item_short = 0, item_long = s.short_items;           // next item index of each kind
    int token_short = 0, token_long = s.num_short_tokens;    // next token index of each kind
    long long cursor = 0;                                    // into `tokens`
    int want_cursor = 0, row = 0;
    // rows keep the caller's order, so the first token of each entry is needed before the rows are written:
    // a first pass places the entries, a second writes the rows
    static thread_local int first_of_entry_small[256];
    int* first_of_entry = n <= 256 ? first_of_entry_small : new int[n];
    for (int i = 0; i < n; ++i) {
        const int c = (int)counts[i];
        const bool is_long = c >= long_entry;
        int& item = is_long ? item_long : item_short;
        int& token = is_long ? token_long : token_short;
        item_slot[item] = (int)slots[i];
        q_start[item] = token;
        first_of_entry[i] = token;
        for (int j = 0; j < c; ++j) {
            const long long id = tokens[cursor + j];
            if (id < 0 || id >= vocab) {
                if (bad_token) *bad_token = id;
                if (n > 256) delete[] first_of_entry;
                return PS_ERR_BAD_ARGUMENT;
            }
            token_ids[token + j] = (int)id;
        }
        cursor += c;
        token += c;
        ++item;
    }
    // padding entries: one with tokens behind each kind (if any), then empty ones, all of the scratch slot
    if (pad) {
        if (s.extra_short > 0) {
            item_slot[item_short] = scratch_slot;
            q_start[item_short] = token_short;
            for (int j = 0; j < s.extra_short; ++j) token_ids[token_short + j] = 0;
            token_short += s.extra_short;
            ++item_short;
        }
        for (; item_short < s.short_items; ++item_short) { item_slot[item_short] = scratch_slot; q_start[item_short] = token_short; }
        if (s.extra_long > 0) {
            item_slot[item_long] = scratch_slot;
            q_start[item_long] = token_long;
            for (int j = 0; j < s.extra_long; ++j) token_ids[token_long + j] = 0;
            token_long += s.extra_long;
            ++item_long;
        }
        for (; item_long < s.I; ++item_long) { item_slot[item_long] = scratch_slot; q_start[item_long] = token_long; }
    }
    q_start[s.I] = s.T;
    for (int i = 0; i < n; ++i)
        for (int w = 0; w < want_counts[i]; ++w) logit_rows[row++] = first_of_entry[i] + wants[want_cursor++];
    const int repeat = row > 0 ? logit_rows[0] : 0;         // padded rows repeat the first one
    for (; row < s.R; ++row) logit_rows[row] = repeat;
    if (n > 256) delete[] first_of_entry;
    return PS_OK;
}
