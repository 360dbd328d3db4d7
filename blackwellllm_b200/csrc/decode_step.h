// bw_decode_step: one decode-only step of the engine behind ONE C call: reconcile the sequences'
// positions, reserve pages and pack the step (the host runtime's bookkeeping), copy the packed step to
// the device, replay the captured graph of this batch size, choose the tokens (greedy) and read them back.
// It is the C face of the step's hot path; configuration, loading and the scheduler's policy stay in Python
// (the reference's public surface is a C++ class with status codes: include/blackwell/engine.h:104-161,
// include/blackwell/engine_status.h:23-57; the names of the codes below follow its EngineStatus).
//
// The caller owns every buffer: the packed step in pinned host memory, the device buffer that the captured
// kernels read (fixed address), the logits the graph writes, the sampled tokens on the device and their
// pinned host copy.  Nothing is allocated here.
#pragma once

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    BW_STEP_SUCCESS = 0,
    BW_STEP_CUDA_RUNTIME_ERROR = 1,   // a CUDA call failed; cuda_error holds its code
    BW_STEP_OUT_OF_PAGES = 2,         // the cache has no pages for this step; nothing was changed
    BW_STEP_INVALID_ARGUMENT = 3,     // a bad token id, a sequence twice, a position outside the context
    BW_STEP_INVALID_CONFIG = 4,       // the packed step does not have the size the graph was captured for
    BW_STEP_STATE_MISMATCH = 5        // a position leaves a gap after the sequence's cached tokens; unknown sequence; not bound
} bw_step_status;

typedef struct {
    void* cache;                  // the host runtime's cache (bwh_create)
    int n;                        // sequences in the step (one token each)
    int* handles;                 // [n] their handles in the host runtime
    const int* tokens;            // [n] host token ids (placeholders 0 if device_tokens is given)
    const int* positions;         // [n] position of each token; below the sequence's length: the sequence is rewound to it
    const int* device_tokens;     // device [n] or null: token ids taken on the device (the previous step's sampled tokens)
    int vocab;
    int table_width;              // block-table entries per sequence that the graph was captured with
    long long max_context;        // positions allowed per sequence
    int* pinned;                  // pinned host buffer for the packed step
    long long pinned_words;
    int* device_step;             // device buffer the captured kernels read; exactly step_words long
    long long step_words;
    void* graph_exec;             // cudaGraphExec_t of this batch size
    void* stream;                 // cudaStream_t
    const float* logits;          // device [n, vocab] (row stride logits_ld): what the graph writes
    long long logits_ld;
    int* sampled_device;          // device [n]
    int* sampled_host;            // pinned host [n]; null: no read-back
    int wait;                     // != 0: return when the tokens are in sampled_host
    int cuda_error;               // out: the failing CUDA call's code
} bw_decode_step_args;

// The host runtime's and the sampler's entry points (addresses of bwh_pack_step, bwh_length, bwh_truncate
// and bw_sample), once per process, before the first step.
int bw_decode_step_bind(void* pack_step, void* length, void* truncate, void* sample);

// One step.  On anything but BW_STEP_SUCCESS no kernel was launched; the sequences may have been rewound to
// the given positions (what the step would have done first), nothing else was changed.
int bw_decode_step(bw_decode_step_args* args);

#ifdef __cplusplus
}
#endif
