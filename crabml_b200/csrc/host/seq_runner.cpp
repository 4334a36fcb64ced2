// seq_runner.cpp -- slots, step and greedy generation shared by every multi-sequence runner (seq_runner.hpp), and their C entry points.
#include "seq_runner.hpp"

using crabml::CudaTensor;
using crabml::TensorError;

int32_t csr_runner::open() {
    int found = -1;
    for (size_t i = 0; i < slots.size(); i++)
        if (!slots[i].live) { found = (int)i; break; }                  // lowest free slot first: closed slots are reused before new ones are made
    if (found < 0) {
        slots.emplace_back();
        found = (int)slots.size() - 1;
        slots[found].state = make_state();
    }
    reset_state(*slots[found].state);
    slots[found].len = 0;
    slots[found].live = true;
    return found;
}
void csr_runner::close(int32_t slot) { slot_ref(slot).live = false; }
int64_t csr_runner::len(int32_t slot) const {
    if (slot < 0 || slot >= (int32_t)slots.size() || !slots[slot].live) return -1;
    return slots[slot].len;
}
void csr_runner::stats(int64_t* out3) const {
    out3[0] = (int64_t)slots.size();
    out3[1] = 0;
    for (auto& s : slots) out3[1] += s.live;
    out3[2] = state_bytes_per_slot;
}

void csr_runner::step(int32_t slot, const int64_t* tokens, int32_t n, const int32_t* want, int32_t n_want, float* out) {
    Slot& s = slot_ref(slot);
    for (int i = 0; i < n; i++)
        if (tokens[i] < 0 || tokens[i] >= vocab) throw TensorError("token id " + std::to_string(tokens[i]) + " is outside the vocabulary");
    for (int i = 0; i < n_want; i++)
        if (want[i] < 0 || want[i] >= n || (i > 0 && want[i] <= want[i - 1])) throw TensorError("wanted positions must be ascending indices into the step's tokens");
    int wi = 0;
    for (int64_t c0 = 0; c0 < n; c0 += chunk) {
        const int64_t cn = std::min<int64_t>(chunk, n - c0);
        CudaTensor x = forward_chunk(*s.state, s.len, tokens + c0, cn, -1);
        s.len += cn;
        std::vector<int64_t> rows;
        while (wi + (int)rows.size() < n_want && want[wi + rows.size()] < c0 + cn) rows.push_back(want[wi + rows.size()] - c0);
        if (!rows.empty()) {
            CudaTensor lg = logits_of(x, rows);
            lg.export_to(out + (size_t)wi * vocab, rows.size() * (size_t)vocab);
            wi += (int)rows.size();
        }
    }
}

void csr_runner::generate_greedy(int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos, int64_t* out_tokens, int32_t* n_out) {
    Slot& s = slot_ref(slot);
    for (int i = 0; i < n_prompt; i++)
        if (prompt[i] < 0 || prompt[i] >= vocab) throw TensorError("token id outside the vocabulary");
    CudaTensor x;
    int64_t last_n = 0;
    for (int64_t c0 = 0; c0 < n_prompt; c0 += chunk) {
        last_n = std::min<int64_t>(chunk, n_prompt - c0);
        x = forward_chunk(*s.state, s.len, prompt + c0, last_n, -1);
        s.len += last_n;
    }
    logits_of(x, {last_n - 1}).reshape({vocab}).argmax_to_slot(0, 0);
    int64_t done = 1;
    if (eos >= 0) check(cc_read_history(dev, 0, 1, out_tokens));
    for (; done < steps; done++) {
        if (eos >= 0 && out_tokens[done - 1] == eos) break;
        x = forward_chunk(*s.state, s.len, nullptr, 1, 0);
        s.len += 1;
        logits_of(x, {0}).reshape({vocab}).argmax_to_slot(0, done);
        if (eos >= 0) check(cc_read_history(dev, done, 1, out_tokens + done));
    }
    if (eos < 0) check(cc_read_history(dev, 0, done, out_tokens));
    *n_out = (int32_t)done;
}

static thread_local std::string g_create_error;
void crabml::seq_set_create_error(const std::string& s) { g_create_error = s; }

extern "C" CC_API const char* csr_last_create_error(void) { return g_create_error.c_str(); }
extern "C" CC_API void csr_runner_destroy(csr_runner* r) { delete r; }
extern "C" CC_API const char* csr_runner_last_error(csr_runner* r) { return r ? r->last_error.c_str() : ""; }
extern "C" CC_API int csr_seq_open(csr_runner* r, int32_t* slot_out) {
    if (!r || !slot_out) return CC_ERR_ARG;
    return crabml::seq_guarded(r, nullptr, [&] { *slot_out = r->open(); });
}
extern "C" CC_API int csr_seq_close(csr_runner* r, int32_t slot) {
    if (!r) return CC_ERR_ARG;
    return crabml::seq_guarded(r, nullptr, [&] { r->close(slot); });
}
extern "C" CC_API int64_t csr_seq_len(csr_runner* r, int32_t slot) { return r ? r->len(slot) : -1; }
extern "C" CC_API int csr_runner_stats(csr_runner* r, int64_t* out3) {
    if (!r || !out3) return CC_ERR_ARG;
    r->stats(out3);
    return CC_OK;
}
extern "C" CC_API int csr_runner_step(csr_runner* r, int32_t slot, const int64_t* tokens, int32_t n_tokens, const int32_t* want, int32_t n_want, float* logits_out) {
    if (!r || !tokens || n_tokens < 1 || n_want < 0 || (n_want > 0 && (!want || !logits_out))) return CC_ERR_ARG;
    return crabml::seq_guarded(r, nullptr, [&] { r->step(slot, tokens, n_tokens, want, n_want, logits_out); });
}
extern "C" CC_API int csr_runner_generate_greedy(csr_runner* r, int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos, int64_t* out_tokens,
                                                 int32_t* n_out) {
    if (!r || !prompt || n_prompt < 1 || steps < 1 || !out_tokens || !n_out) return CC_ERR_ARG;
    *n_out = 0;
    return crabml::seq_guarded(r, nullptr, [&] { r->generate_greedy(slot, prompt, n_prompt, steps, eos, out_tokens, n_out); });
}
