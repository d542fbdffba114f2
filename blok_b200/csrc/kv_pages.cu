// Host-side bookkeeping of the paged latent cache: which pages of the pool every sequence slot holds.
// The reference keeps one contiguous KV region per layer and refuses a sequence longer than the region
// (KvCache, src/kimi_exec.cu:192-238, capacity check :205); with pages, sequences of different lengths share one pool
// and a finished sequence returns its pages.  One page number addresses the same page in every layer's pool, so one
// table serves the whole model.  Nothing here touches the GPU except blok_kv_pages_upload.
#include <cstring>
#include <new>
#include <vector>

#include "common.cuh"

struct blok_kv_pages {
  int n_pages = 0, page_rows = 0, slots = 0, table_stride = 0;
  std::vector<int> table;      // [slots, table_stride] page numbers; entries past a slot's count are 0
  std::vector<int> count;      // pages held by each slot
  std::vector<int> refs;       // slots holding each page (a forked prefix is shared)
  std::vector<int> free_list;  // pages with refs == 0, handed out from the back
  bool dirty = true;           // the table changed since the last upload
};

extern "C" int blok_kv_pages_create(int n_pages, int page_rows, int slots, int table_stride, blok_kv_pages_t **out) {
  BLOK_REQUIRE(out, BLOK_ERR_ARG, "blok_kv_pages_create: null pointer");
  BLOK_REQUIRE(n_pages >= 1 && slots >= 1 && table_stride >= 1 && page_rows >= 32 && page_rows % 32 == 0, BLOK_ERR_SHAPE,
               "blok_kv_pages_create: need pages, slots, table_stride >= 1 and page_rows a positive multiple of 32 (got %d, %d, %d, %d)",
               n_pages, slots, table_stride, page_rows);
  blok_kv_pages *p = new (std::nothrow) blok_kv_pages();
  BLOK_REQUIRE(p, BLOK_ERR_ARG, "blok_kv_pages_create: out of host memory");
  p->n_pages = n_pages;
  p->page_rows = page_rows;
  p->slots = slots;
  p->table_stride = table_stride;
  p->table.assign((size_t)slots * table_stride, 0);
  p->count.assign(slots, 0);
  p->refs.assign(n_pages, 0);
  p->free_list.resize(n_pages);
  for (int i = 0; i < n_pages; ++i) p->free_list[i] = n_pages - 1 - i;  // page 0 is handed out first
  *out = p;
  return BLOK_OK;
}

extern "C" int blok_kv_pages_destroy(blok_kv_pages_t *p) {
  delete p;
  return BLOK_OK;
}

static int check_slot(const blok_kv_pages *p, int slot, const char *who) {
  BLOK_REQUIRE(p, BLOK_ERR_ARG, "%s: null handle", who);
  BLOK_REQUIRE(slot >= 0 && slot < p->slots, BLOK_ERR_ARG, "%s: slot %d outside [0, %d)", who, slot, p->slots);
  return BLOK_OK;
}

extern "C" int blok_kv_pages_reserve(blok_kv_pages_t *p, int slot, long n_rows) {
  if (int rc = check_slot(p, slot, "blok_kv_pages_reserve")) return rc;
  BLOK_REQUIRE(n_rows >= 0, BLOK_ERR_ARG, "blok_kv_pages_reserve: negative row count");
  const long need = (n_rows + p->page_rows - 1) / p->page_rows;
  BLOK_REQUIRE(need <= p->table_stride, BLOK_ERR_SHAPE, "blok_kv_pages_reserve: %ld rows need %ld pages, a slot holds at most %d",
               n_rows, need, p->table_stride);
  const int have = p->count[slot];
  if (need <= have) return BLOK_OK;  // a reservation only grows
  BLOK_REQUIRE((long)p->free_list.size() >= need - have, BLOK_ERR_WORKSPACE,
               "blok_kv_pages_reserve: the pool has %zu free pages, slot %d needs %ld more", p->free_list.size(), slot, need - have);
  int *row = p->table.data() + (size_t)slot * p->table_stride;
  for (long j = have; j < need; ++j) {
    const int page = p->free_list.back();
    p->free_list.pop_back();
    p->refs[page] = 1;
    row[j] = page;
  }
  p->count[slot] = (int)need;
  p->dirty = true;
  return BLOK_OK;
}

extern "C" int blok_kv_pages_release(blok_kv_pages_t *p, int slot) {
  if (int rc = check_slot(p, slot, "blok_kv_pages_release")) return rc;
  int *row = p->table.data() + (size_t)slot * p->table_stride;
  for (int j = 0; j < p->count[slot]; ++j) {
    if (--p->refs[row[j]] == 0) p->free_list.push_back(row[j]);
    row[j] = 0;
  }
  if (p->count[slot]) p->dirty = true;
  p->count[slot] = 0;
  return BLOK_OK;
}

extern "C" int blok_kv_pages_fork(blok_kv_pages_t *p, int src_slot, int dst_slot, long n_rows) {
  if (int rc = check_slot(p, src_slot, "blok_kv_pages_fork")) return rc;
  if (int rc = check_slot(p, dst_slot, "blok_kv_pages_fork")) return rc;
  BLOK_REQUIRE(src_slot != dst_slot && p->count[dst_slot] == 0, BLOK_ERR_STATE,
               "blok_kv_pages_fork: the destination slot must be another, empty slot");
  BLOK_REQUIRE(n_rows >= 0 && n_rows % p->page_rows == 0 && n_rows / p->page_rows <= p->count[src_slot], BLOK_ERR_SHAPE,
               "blok_kv_pages_fork: only whole pages the source holds can be shared (%ld rows, page %d rows, source holds %d pages)",
               n_rows, p->page_rows, p->count[src_slot]);
  const int n = (int)(n_rows / p->page_rows);
  const int *src = p->table.data() + (size_t)src_slot * p->table_stride;
  int *dst = p->table.data() + (size_t)dst_slot * p->table_stride;
  for (int j = 0; j < n; ++j) {
    dst[j] = src[j];
    ++p->refs[src[j]];
  }
  p->count[dst_slot] = n;
  if (n) p->dirty = true;
  return BLOK_OK;
}

extern "C" int blok_kv_pages_free_count(const blok_kv_pages_t *p) { return p ? (int)p->free_list.size() : 0; }

extern "C" long blok_kv_pages_rows(const blok_kv_pages_t *p, int slot) {
  return (p && slot >= 0 && slot < p->slots) ? (long)p->count[slot] * p->page_rows : 0;
}

extern "C" const int *blok_kv_pages_table(const blok_kv_pages_t *p) { return p ? p->table.data() : nullptr; }

extern "C" int blok_kv_pages_upload(blok_kv_pages_t *p, int *device_table, blok_stream_t stream) {
  BLOK_REQUIRE(p && device_table, BLOK_ERR_ARG, "blok_kv_pages_upload: null pointer");
  if (!p->dirty) return BLOK_OK;
  // The host table is pageable memory: the runtime stages the copy before this call returns, so the table may
  // change again at once.
  BLOK_CUDA(cudaMemcpyAsync(device_table, p->table.data(), p->table.size() * sizeof(int), cudaMemcpyHostToDevice,
                            (cudaStream_t)stream));
  p->dirty = false;
  return BLOK_OK;
}
