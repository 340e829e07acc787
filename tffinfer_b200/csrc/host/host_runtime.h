// Host side of a step, in C++: the page pools, the block tables of the live requests, the state slots,
// and the packing of a step's integer arrays (token rows, per-request arrays, request order, padded block
// tables) into the one buffer that is copied to the device.  No CUDA in here: the library builds with the
// host compiler alone and is loaded by tffinfer_b200/cache/native.py through ctypes.
//
// Reference counterpart: LLMKVCache / PageManager / LayerKVContext (src/core/runtime/KVCache.h:36-473) and
// the flat LLMBatch of LLMBatchManager (src/core/runtime/BatchManager.h:77-99).  What differs is said in
// tffinfer_b200/cache/manager.py, whose Python classes are the plain twin of this file: same interface,
// same decisions, compared under random orders of requests by the tests.
//
// Every function returns >= 0 on success and a negative TFFH_ERR_* otherwise; tffh_last_error gives the
// words.  Requests are named by 64-bit handles that the caller chooses.
#pragma once
#include <cstdint>

#if defined(__GNUC__)
#define TFFH_API extern "C" __attribute__((visibility("default")))
#else
#define TFFH_API extern "C"
#endif

enum {
    TFFH_ERR_ARGUMENT = -1,      // a bad size, group or pointer
    TFFH_ERR_UNKNOWN = -2,       // the request is not live
    TFFH_ERR_LIVE = -3,          // the request is live already
    TFFH_ERR_ACCOUNTING = -4,    // a page or slot freed twice, held twice, lost, or tokens committed beyond the reserved
    TFFH_ERR_TOO_SMALL = -5,     // the caller's buffer is too small
    TFFH_ERR_DUPLICATE = -6,     // a request appears twice in one step
    TFFH_ERR_TOO_LONG = -7,      // a request would grow beyond the longest sequence allowed
};

// ---- cache manager
TFFH_API void* tffh_cache_create(int num_groups, const int* windows, int page_size, const int* pages_per_group,
                                 int max_live_requests);
TFFH_API void tffh_cache_destroy(void* cache);
TFFH_API const char* tffh_last_error(void* cache);

TFFH_API int tffh_admit(void* cache, int64_t req);                    // the slot, or -100 when no slot is free
TFFH_API int tffh_is_live(void* cache, int64_t req);
TFFH_API int tffh_num_tokens(void* cache, int64_t req);
TFFH_API int tffh_slot_of(void* cache, int64_t req);
TFFH_API int tffh_pages_needed(void* cache, int64_t req, int n_new, int* per_group);
TFFH_API int tffh_reserve(void* cache, int64_t req, int n_new);       // 1 taken, 0 not enough pages (nothing taken)
TFFH_API int tffh_commit(void* cache, int64_t req, int n_new);
TFFH_API int tffh_release(void* cache, int64_t req);
TFFH_API int tffh_block_table(void* cache, int64_t req, int group, int* out, int capacity);   // its length
TFFH_API int tffh_check(void* cache);                                 // 0 when the accounts are right

// what: 0 pages in all, 1 free pages, 2 most pages ever taken (group is the pool);
//       3 free slots, 4 live requests (group ignored)
TFFH_API int tffh_count(void* cache, int what, int group);

// ---- a whole step at once
// Checks the requests of a step (live, each once, at least one token, not beyond max_model_len when that is
// > 0) and takes the pages that all of them need, in every group, or none at all.  Returns 1 when the pages
// were taken; 0 when they do not suffice (detail: group, pages needed, pages free; nothing taken); a negative
// error with detail[0] = the index of the request it is about.
TFFH_API int tffh_reserve_step(void* cache, int n, const int64_t* reqs, const int* q_lens, int max_model_len,
                               int* detail);
// counts[i] tokens of request reqs[i] were written (tffh_commit for each).
TFFH_API int tffh_commit_step(void* cache, int n, const int64_t* reqs, const int* counts);

// ---- packing a step
// Requests reqs[0..n) bring q_lens[i] tokens each (tokens: all of them, flat); want_start[i]..want_start[i+1]
// of ``want`` are the places among request i's tokens whose logits are asked for; tok_src (or null) gives per
// token the row of the previous step's drawn tokens to take the id from, or -1.  With pad_requests > n the
// batch is filled up with requests of one token 0 at position 0 that write to dummy_pages / dummy_slot and
// whose logits are asked for.  widths[g]: block-table width of group g (<= 0: the widest table, at least 1;
// the width chosen is written back; a table wider than a width given is TFFH_ERR_ARGUMENT).  ``out``
// receives, in this order: token ids, positions, request row of each token, first row of each request
// (B + 1), first position, tokens in the cache after the step, slots, wanted rows (R), request order (by
// new tokens, then longest context first), tok_src (T), and one [B, width] block table a group.  info: T, B, R, longest portion, longest context, 1 if any token has a source row,
// 1 if every real request brings one token, real wanted rows.  Returns the number of int32 written, or
// TFFH_ERR_TOO_SMALL with the number needed in info[0] when out_capacity is smaller (out may be null then).
TFFH_API int64_t tffh_pack_step(void* cache, int n, const int64_t* reqs, const int* q_lens, const int* tokens,
                                const int* want_start, const int* want, const int* tok_src,
                                int pad_requests, int* widths, const int* dummy_pages, int dummy_slot,
                                int* out, int64_t out_capacity, int* info);

// ---- planning a step (the decisions of engine/scheduler.py: Scheduler.schedule, its Python twin)
// running[0..n_running): the live requests in the order of their admission, with their lengths (prompt +
// generated tokens); waiting[0..n_waiting): the queue in arrival order, with the handle each would be admitted
// under, its length and the length of its prompt.  Decoded tokens first (one each), then portions of prompts
// under budget_tokens, then admissions while a slot, budget and pages are there; when the pages do not
// suffice the request admitted last is released and goes to the front of the queue (alone, it ends: out of
// memory) and the pass starts again.  Pages of the chosen requests are taken.  Writes events of four ints
// (kind, uid, a, b), uid being the index into running[] or n_running + the index into waiting[], in the order
// in which they happened, and returns their number:
//   TFFH_EVENT_PREEMPT  uid                      released, now first in the queue
//   TFFH_EVENT_FINISH   uid, reason, was_running ended without running (released if it was running)
//   TFFH_EVENT_ADMIT    uid, slot                 now live
//   TFFH_EVENT_RUN      uid, tokens, start        brings ``tokens`` tokens from position ``start`` in this step
enum { TFFH_EVENT_PREEMPT = 1, TFFH_EVENT_FINISH = 2, TFFH_EVENT_ADMIT = 3, TFFH_EVENT_RUN = 4 };
enum { TFFH_REASON_OUT_OF_MEMORY = 1, TFFH_REASON_TOO_LONG = 2, TFFH_REASON_EMPTY_PROMPT = 3 };
TFFH_API int tffh_plan_step(void* cache, int budget_tokens, int max_model_len,
                            int n_running, const int64_t* running, const int* running_len,
                            int n_waiting, const int64_t* waiting, const int* waiting_len, const int* waiting_prompt_len,
                            int* events, int capacity);
