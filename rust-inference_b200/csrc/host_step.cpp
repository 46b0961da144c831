// The host side of a step: checks what the sequences bring and writes the step's int32 tables,
// which one copy then takes to the device.
//
// A step packs its tokens back to back, sequence after sequence (nothing is padded).  The tables,
// in this order in one buffer:
//   ids [T], tok_seq [T] (which sequence of the step a token belongs to), tok_pos [T] (its position
//   in that sequence: the cache's length before the step plus its place), want_rows [W] (the packed
//   rows whose logits are asked for), seq_slot [B], seq_start [B + 1] (first packed row of each
//   sequence, then T), seq_len [B] (length after the step).
// Positions come from the cache's lengths, so they cannot disagree with the cache (in
// thanhauco/rust-inference they are a separate argument of forward, src/models/mod.rs:36-44).
//
// Plain C functions; a non-zero return code means that nothing was written and `ri_last_error()`
// holds the message.
#include <cstdarg>
#include <cstdint>
#include <cstdio>

static thread_local char ri_errbuf[512];
extern "C" const char* ri_last_error() { return ri_errbuf; }

static int fail(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(ri_errbuf, sizeof(ri_errbuf), fmt, ap);
    va_end(ap);
    return 1;
}

extern "C" {

// What B sequences bring: n_new[b] tokens each (ids in `tokens`, back to back) and n_want[b] wanted
// places (in `wants`, back to back, each a place among that sequence's own tokens).  Checks all of
// it and gives T and W.  Nothing else happens here: a step that fails this check has not touched
// the cache.
int ri_step_check(int B, const int* slots, const int* n_new, const long long* tokens, long long vocab, const int* n_want,
                  const int* wants, long long* T_out, long long* W_out) {
    if (B <= 0) return fail("a step needs at least one sequence");
    long long T = 0, W = 0;
    for (int b = 0; b < B; b++) {
        if (n_new[b] <= 0) return fail("slot %d brings no token", slots[b]);
        for (int i = 0; i < n_new[b]; i++) {
            const long long id = tokens[T + i];
            if (id < 0 || id >= vocab) return fail("slot %d: token id outside the vocabulary of %lld", slots[b], vocab);
        }
        for (int i = 0; i < n_want[b]; i++) {
            const int w = wants[W + i];
            if (w < 0 || w >= n_new[b]) return fail("slot %d: wanted place outside its %d tokens", slots[b], n_new[b]);
        }
        T += n_new[b];
        W += n_want[b];
    }
    if (T >= (1ll << 31) || W >= (1ll << 31)) return fail("a step of %lld tokens", T);
    *T_out = T;
    *W_out = W;
    return 0;
}

// Writes the tables of a checked step into `out` (T + T + T + W + B + B + 1 + B int32).  `before`: each
// sequence's length in the cache before the step.  Gives the most tokens one sequence brings and the
// longest sequence after the step.
void ri_step_fill(int B, const int* slots, const int* before, const int* n_new, const long long* tokens, const int* n_want,
                  const int* wants, long long T, long long W, int32_t* out, int* max_new_out, int* max_len_out) {
    int32_t* ids = out;
    int32_t* tok_seq = ids + T;
    int32_t* tok_pos = tok_seq + T;
    int32_t* want_rows = tok_pos + T;
    int32_t* seq_slot = want_rows + W;
    int32_t* seq_start = seq_slot + B;
    int32_t* seq_len = seq_start + B + 1;
    long long t0 = 0, w0 = 0;
    int max_new = 0, max_len = 0;
    for (int b = 0; b < B; b++) {
        const int n = n_new[b];
        for (int i = 0; i < n; i++) {
            ids[t0 + i] = (int32_t)tokens[t0 + i];
            tok_seq[t0 + i] = b;
            tok_pos[t0 + i] = before[b] + i;
        }
        for (int i = 0; i < n_want[b]; i++) want_rows[w0 + i] = (int32_t)(t0 + wants[w0 + i]);
        seq_slot[b] = slots[b];
        seq_start[b] = (int32_t)t0;
        seq_len[b] = before[b] + n;
        if (n > max_new) max_new = n;
        if (before[b] + n > max_len) max_len = before[b] + n;
        t0 += n;
        w0 += n_want[b];
    }
    seq_start[B] = (int32_t)T;
    *max_new_out = max_new;
    *max_len_out = max_len;
}

// A decode step brings one token per sequence: the check of its ids (before the cache grows).
int ri_step_check_decode(int B, const long long* tokens, long long vocab) {
    if (B <= 0) return fail("a step needs at least one sequence");
    for (int b = 0; b < B; b++)
        if (tokens[b] < 0 || tokens[b] >= vocab) return fail("token id outside the vocabulary of %lld", vocab);
    return 0;
}

// The tables of a decode step, in which every sequence brings one token and wants its logits:
// T = W = B.  `tokens` may be null when the ids are already on the device (they are copied there
// after the tables); the columns that are the same for every step of B sequences (tok_seq,
// want_rows, seq_start) are written when `constants` is set.  Gives the longest sequence after the step.
void ri_step_fill_decode(int B, const int* slots, const int* before, const long long* tokens, int constants, int32_t* out,
                         int* max_len_out) {
    int32_t* ids = out;
    int32_t* tok_seq = ids + B;
    int32_t* tok_pos = tok_seq + B;
    int32_t* want_rows = tok_pos + B;
    int32_t* seq_slot = want_rows + B;
    int32_t* seq_start = seq_slot + B;
    int32_t* seq_len = seq_start + B + 1;
    int max_len = 0;
    for (int b = 0; b < B; b++) {
        ids[b] = tokens ? (int32_t)tokens[b] : 0;
        tok_pos[b] = before[b];
        seq_slot[b] = slots[b];
        seq_len[b] = before[b] + 1;
        if (before[b] + 1 > max_len) max_len = before[b] + 1;
        if (constants) {
            tok_seq[b] = b;
            want_rows[b] = b;
            seq_start[b] = b;
        }
    }
    if (constants) seq_start[B] = B;
    *max_len_out = max_len;
}

}  // extern "C"
