// seq_runner.hpp -- the part of a multi-sequence model runner that does not depend on the model family: sequence slots (taken, reset,
// given back, reused lowest first), the step function (token and index checks, passes of at most `chunk` tokens, logits of the wanted
// places), and greedy generation with sampling on the device.  A family (zatorax_runner.cpp, meresun_runner.cpp) derives from
// csr_runner and supplies its per-sequence state and one pass over a run of tokens.  The C entry points are in seq_runner.cpp.
#pragma once

#include <algorithm>
#include <memory>
#include <string>
#include <vector>

#include "../../../include/crabml_seqrunner.h"
#include "cuda_tensor.hpp"

namespace crabml {
// what one sequence holds between steps; each family derives its own
struct SeqState {
    virtual ~SeqState() = default;
};
}  // namespace crabml

struct csr_runner {
    cc_device* dev = nullptr;
    int32_t width = 0, vocab = 0, chunk = 256;
    int64_t state_bytes_per_slot = 0;
    std::string last_error;

    virtual ~csr_runner() = default;

    int32_t open();
    void close(int32_t slot);
    int64_t len(int32_t slot) const;
    void stats(int64_t* out3) const;
    void step(int32_t slot, const int64_t* tokens, int32_t n, const int32_t* want, int32_t n_want, float* out);
    void generate_greedy(int32_t slot, const int64_t* prompt, int32_t n_prompt, int32_t steps, int64_t eos, int64_t* out_tokens, int32_t* n_out);

    void check(int rc) { crabml::CudaTensor::check(dev, rc); }
    crabml::CudaTensor adopt(cc_buf* b, std::vector<int64_t> shape) { return crabml::CudaTensor(dev, b, crabml::TensorStrider(std::move(shape))); }

protected:
    struct Slot {
        std::unique_ptr<crabml::SeqState> state;
        int64_t len = 0;
        bool live = false;
    };
    std::vector<Slot> slots;
    Slot& slot_ref(int32_t slot) {
        if (slot < 0 || slot >= (int32_t)slots.size() || !slots[slot].live) throw crabml::TensorError("sequence slot " + std::to_string(slot) + " is not open");
        return slots[slot];
    }

    // ---- what a family supplies ---------------------------------------------------------------------------------------------------
    virtual std::unique_ptr<crabml::SeqState> make_state() = 0;
    // a reused slot must start like a new one
    virtual void reset_state(crabml::SeqState& s) = 0;
    // one pass over n <= chunk tokens at positions pos0 .. (token ids from `tokens`, or from device slot `device_slot` when >= 0);
    // returns the residual stream [n, width] after the last layer
    virtual crabml::CudaTensor forward_chunk(crabml::SeqState& s, int64_t pos0, const int64_t* tokens, int64_t n, int device_slot) = 0;
    // final norm and head of the given rows of x -> [rows, vocab]
    virtual crabml::CudaTensor logits_of(const crabml::CudaTensor& x, const std::vector<int64_t>& rows) = 0;
};

namespace crabml {
// runs f, turning exceptions into status codes and the runner's last_error (r may be NULL while a runner is being created)
template <class F>
int seq_guarded(csr_runner* r, std::string* err, F&& f) {
    try {
        f();
        return CC_OK;
    } catch (const TensorError& e) {
        if (r) r->last_error = e.what();
        if (err) *err = e.what();
        return CC_ERR_TENSOR;
    } catch (const std::exception& e) {
        if (r) r->last_error = e.what();
        if (err) *err = e.what();
        return CC_ERR_ARG;
    }
}
// the text csr_last_create_error returns
void seq_set_create_error(const std::string& s);
}  // namespace crabml
