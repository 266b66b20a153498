// layerprog.h — internal interface between engine.cu (the C ABI, the sequence slots, the batch scheduler) and layerprog.cu (the
// layer-program models: a decoder given as a list of layers with their own token mixers).  Every function returns a b200_status;
// `err` receives the message.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include <string>

#include "../../include/llama_b200.h"

struct LpModel;

int lp_create(const b200_program_desc* prog, const b200_layer_desc* layers, int device, cudaStream_t stream, bool taps, LpModel** out,
              std::string* err);
int lp_upload(LpModel* m, const char* name, uint32_t ggml_type, const uint64_t* ne, int n_dims, const void* host, size_t nbytes,
              std::string* err);
int lp_finalize(LpModel* m, std::string* err);
void lp_destroy(LpModel* m);
// One batch of token runs.  pos0[i] is the number of tokens slot seqs[i] already holds.  Exactly one of logits_out (n_want x vocab,
// host) and pick_out (n_want greedy picks, host; last maximum wins) may be non-null; both null runs the tokens for their state only.
int lp_step(LpModel* m, int n_runs, const int* seqs, const int* pos0, const int* lens, const uint32_t* tokens, const int* want_rows,
            int n_want, float* logits_out, uint32_t* pick_out, std::string* err);
// The slot's cache and state go back to the pool; its next token starts a new sequence.
int lp_release(LpModel* m, int seq, std::string* err);
int lp_layer_runs(const LpModel* m);
int lp_get_taps(LpModel* m, float* out, size_t cap_floats, std::string* err);
// statistics: kernels launched so far, bytes of weights one token reads, cache bytes one position holds
void lp_stats(const LpModel* m, uint64_t* launches, uint64_t* weight_bytes, uint64_t* kv_bytes_per_pos);
// slots that currently own memory / blocks waiting in the pool (tests of the slot manager)
void lp_pool_counts(const LpModel* m, int* live, int* pooled);
