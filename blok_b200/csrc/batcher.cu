// Continuous batching, host side: which queued request enters which sequence slot, which slots step in the next
// iteration, and when a sequence ends.  The reference serves one prompt per process (generate(), src/kimi_exec.cu:
// 780-893: replay the prompt, then one token per iteration until EOS or the token budget, :887-890); this keeps that
// per-sequence rule and runs up to `slots` sequences side by side over one page pool.
//
// Admission is first come, first served and reserves to the maximum: a request enters only when a slot is free and
// the pool can hold its prompt plus its whole token budget next to the budgets already admitted, so a running
// sequence never finds the pool empty and nothing is ever evicted.  No GPU and no CUDA call in this file.
#include <deque>
#include <new>
#include <vector>

#include "common.cuh"

namespace {
struct Request {
  int n_prompt = 0, max_new = 0;
  int emitted = 0;
  int slot = -1;       // -1: waiting or finished
  bool done = false;
  bool prefilled = false;
  long pages = 0;      // pages committed for prompt + budget
};
}  // namespace

struct blok_batcher {
  int slots = 0, n_pages = 0, page_rows = 0, max_ctx = 0;
  long committed = 0;                // pages promised to the admitted requests
  std::vector<Request> requests;     // by request id
  std::deque<int> waiting;           // request ids in arrival order
  std::vector<int> slot_request;     // request in each slot, -1 when free
  int unfinished = 0;
};

extern "C" int blok_batcher_create(int slots, int n_pages, int page_rows, int max_ctx, blok_batcher_t **out) {
  BLOK_REQUIRE(out, BLOK_ERR_ARG, "blok_batcher_create: null pointer");
  BLOK_REQUIRE(slots >= 1 && n_pages >= 1 && page_rows >= 1 && max_ctx >= 1, BLOK_ERR_SHAPE,
               "blok_batcher_create: slots, pages, page_rows and max_ctx must be positive");
  blok_batcher *b = new (std::nothrow) blok_batcher();
  BLOK_REQUIRE(b, BLOK_ERR_ARG, "blok_batcher_create: out of host memory");
  b->slots = slots;
  b->n_pages = n_pages;
  b->page_rows = page_rows;
  b->max_ctx = max_ctx;
  b->slot_request.assign(slots, -1);
  *out = b;
  return BLOK_OK;
}

extern "C" int blok_batcher_destroy(blok_batcher_t *b) {
  delete b;
  return BLOK_OK;
}

extern "C" int blok_batcher_submit(blok_batcher_t *b, int n_prompt, int max_new, int *request_id) {
  BLOK_REQUIRE(b && request_id, BLOK_ERR_ARG, "blok_batcher_submit: null pointer");
  BLOK_REQUIRE(n_prompt >= 1 && max_new >= 1, BLOK_ERR_ARG, "blok_batcher_submit: empty prompt or max_new < 1");
  BLOK_REQUIRE((long)n_prompt + max_new <= b->max_ctx, BLOK_ERR_SHAPE,
               "blok_batcher_submit: requested sequence exceeds the context (%d)", b->max_ctx);  // :784
  Request r;
  r.n_prompt = n_prompt;
  r.max_new = max_new;
  r.pages = ((long)n_prompt + max_new + b->page_rows - 1) / b->page_rows;
  BLOK_REQUIRE(r.pages <= b->n_pages, BLOK_ERR_WORKSPACE, "blok_batcher_submit: the request needs %ld pages, the pool has %d", r.pages,
               b->n_pages);
  *request_id = (int)b->requests.size();
  b->requests.push_back(r);
  b->waiting.push_back(*request_id);
  ++b->unfinished;
  return BLOK_OK;
}

extern "C" int blok_batcher_plan(blok_batcher_t *b, int *admit_slots, int *admit_requests, int *n_admit, int *decode_slots,
                                 int *n_decode) {
  BLOK_REQUIRE(b && admit_slots && admit_requests && n_admit && decode_slots && n_decode, BLOK_ERR_ARG,
               "blok_batcher_plan: null pointer");
  *n_admit = *n_decode = 0;
  // the sequences already running step once more
  for (int s = 0; s < b->slots; ++s)
    if (b->slot_request[s] >= 0 && b->requests[b->slot_request[s]].prefilled) decode_slots[(*n_decode)++] = s;
  // arrivals enter in order while a slot and the pages for their whole budget are free; the first that does not
  // fit keeps the ones behind it waiting (no overtaking)
  while (!b->waiting.empty()) {
    Request &r = b->requests[b->waiting.front()];
    if (b->committed + r.pages > b->n_pages) break;
    int slot = -1;
    for (int s = 0; s < b->slots && slot < 0; ++s)
      if (b->slot_request[s] < 0) slot = s;
    if (slot < 0) break;
    r.slot = slot;
    b->slot_request[slot] = b->waiting.front();
    b->committed += r.pages;
    admit_slots[*n_admit] = slot;
    admit_requests[*n_admit] = b->waiting.front();
    ++*n_admit;
    b->waiting.pop_front();
  }
  return BLOK_OK;
}

extern "C" int blok_batcher_token(blok_batcher_t *b, int slot, int is_eos, int *finished) {
  BLOK_REQUIRE(b && finished, BLOK_ERR_ARG, "blok_batcher_token: null pointer");
  BLOK_REQUIRE(slot >= 0 && slot < b->slots && b->slot_request[slot] >= 0, BLOK_ERR_STATE, "blok_batcher_token: slot %d holds no sequence",
               slot);
  Request &r = b->requests[b->slot_request[slot]];
  r.prefilled = true;            // the first token of a sequence is the one sampled after its prompt
  if (!is_eos) ++r.emitted;      // EOS ends the sequence and is not emitted (:887)
  *finished = (is_eos || r.emitted >= r.max_new) ? 1 : 0;
  if (*finished) {
    r.done = true;
    r.slot = -1;
    b->committed -= r.pages;
    b->slot_request[slot] = -1;
    --b->unfinished;
  }
  return BLOK_OK;
}

extern "C" int blok_batcher_unfinished(const blok_batcher_t *b) { return b ? b->unfinished : 0; }
extern "C" int blok_batcher_waiting(const blok_batcher_t *b) { return b ? (int)b->waiting.size() : 0; }
extern "C" long blok_batcher_committed_pages(const blok_batcher_t *b) { return b ? b->committed : 0; }
extern "C" int blok_batcher_emitted(const blok_batcher_t *b, int request_id) {
  return (b && request_id >= 0 && request_id < (int)b->requests.size()) ? b->requests[request_id].emitted : -1;
}
