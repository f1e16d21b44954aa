// Host-side bookkeeping of the paged cache, in C++: the block allocator, per-request block
// tables, and the packer that turns one step's rows into the flat int32 arena the kernels read.
//
// The allocator keeps the contract of miniserve/cache/block_allocator.py:1-107 (also
// minicore/src/block_allocator.cpp): a fresh allocator hands out 0, 1, 2, ...; freed blocks go on
// top of a stack and are reused first; allocate is all-or-nothing; free validates the whole call
// before anything changes. Tables follow miniserve/cache/block_table.py:19-89 (blocks_needed,
// append_tokens, slot, rewind, release), with one addition the reference has no use for: a table
// can give back the pages that lie wholly below a position (for layers that only look a window
// back); their entries read -1 afterwards. The packer stands where the reference packs block
// tables for FlashInfer (miniserve/cache/packing.py:25-56, minicore/src/packing.cpp) and builds
// ids/positions in Python (miniserve/engine/model_runner.py:232-249): here one call fills
// everything a step needs.
#include <stdint.h>

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <unordered_map>
#include <vector>

#define MS_EXPORT extern "C" __attribute__((visibility("default")))

namespace ms {
inline char* error_buffer() {
  static thread_local char buf[1024];
  return buf;
}
}  // namespace ms

MS_EXPORT const char* ms_host_last_error() { return ms::error_buffer(); }

namespace {

enum Rc : int { OK = 0, VALUE_ERROR = 1, OUT_OF_BLOCKS = 2, INDEX_ERROR = 3 };

template <typename... A>
int err(int rc, const char* fmt, A... a) {
  snprintf(ms::error_buffer(), 1024, fmt, a...);
  return rc;
}

struct Allocator {
  int num_blocks, block_size;
  std::vector<int> free_stack;  // back() is handed out next
  std::vector<int> ref;
};

struct Table {
  Allocator* alloc;
  std::vector<int> blocks;  // -1: given back because the window has passed it
  long long num_tokens = 0;
  int first_live = 0;  // blocks[0 .. first_live) are -1
};

}  // namespace

// ------------------------------------------------------------------ allocator
MS_EXPORT void* ms_alloc_create(int num_blocks, int block_size) {
  if (num_blocks < 1 || block_size < 1) {
    err(VALUE_ERROR, "num_blocks and block_size must be positive, got %d, %d", num_blocks, block_size);
    return nullptr;
  }
  auto* a = new Allocator{num_blocks, block_size, {}, std::vector<int>(num_blocks, 0)};
  a->free_stack.resize(num_blocks);
  for (int i = 0; i < num_blocks; ++i) a->free_stack[i] = num_blocks - 1 - i;
  return a;
}
MS_EXPORT void ms_alloc_destroy(void* h) { delete static_cast<Allocator*>(h); }
MS_EXPORT int ms_alloc_num_free(void* h) { return (int)static_cast<Allocator*>(h)->free_stack.size(); }
MS_EXPORT int ms_alloc_num_blocks(void* h) { return static_cast<Allocator*>(h)->num_blocks; }
MS_EXPORT int ms_alloc_block_size(void* h) { return static_cast<Allocator*>(h)->block_size; }

MS_EXPORT int ms_alloc_refcount(void* h, int block, int* out) {
  auto* a = static_cast<Allocator*>(h);
  if (block < 0 || block >= a->num_blocks) return err(INDEX_ERROR, "block id %d out of range [0, %d)", block, a->num_blocks);
  *out = a->ref[block];
  return OK;
}

MS_EXPORT int ms_alloc_allocate(void* h, int n, int* out) {
  auto* a = static_cast<Allocator*>(h);
  if (n < 0) return err(VALUE_ERROR, "cannot allocate %d blocks", n);
  if (n > (int)a->free_stack.size()) return err(OUT_OF_BLOCKS, "requested %d blocks, %d free", n, (int)a->free_stack.size());
  for (int i = 0; i < n; ++i) {
    const int b = a->free_stack.back();
    a->free_stack.pop_back();
    a->ref[b] = 1;
    out[i] = b;
  }
  return OK;
}

MS_EXPORT int ms_alloc_incref(void* h, const int* blocks, int n) {
  auto* a = static_cast<Allocator*>(h);
  for (int i = 0; i < n; ++i) {
    if (blocks[i] < 0 || blocks[i] >= a->num_blocks) return err(INDEX_ERROR, "block id %d out of range [0, %d)", blocks[i], a->num_blocks);
    if (a->ref[blocks[i]] == 0) return err(VALUE_ERROR, "incref of free block %d", blocks[i]);
  }
  for (int i = 0; i < n; ++i) a->ref[blocks[i]] += 1;
  return OK;
}

MS_EXPORT int ms_alloc_free(void* h, const int* blocks, int n) {
  auto* a = static_cast<Allocator*>(h);
  std::unordered_map<int, int> drops;
  for (int i = 0; i < n; ++i) {
    if (blocks[i] < 0 || blocks[i] >= a->num_blocks) return err(INDEX_ERROR, "block id %d out of range [0, %d)", blocks[i], a->num_blocks);
    drops[blocks[i]] += 1;
  }
  for (auto& kv : drops)
    if (a->ref[kv.first] < kv.second)
      return err(VALUE_ERROR, "free of block %d: %d releases but reference count %d", kv.first, kv.second, a->ref[kv.first]);
  for (int i = 0; i < n; ++i)
    if (--a->ref[blocks[i]] == 0) a->free_stack.push_back(blocks[i]);
  return OK;
}

// 0 if the free stack and the reference counts describe the same set.
MS_EXPORT int ms_alloc_check(void* h) {
  auto* a = static_cast<Allocator*>(h);
  std::vector<char> seen(a->num_blocks, 0);
  for (int b : a->free_stack) {
    if (b < 0 || b >= a->num_blocks) return err(VALUE_ERROR, "free stack holds invalid block %d", b);
    if (seen[b]) return err(VALUE_ERROR, "duplicate block %d in free stack", b);
    seen[b] = 1;
  }
  for (int b = 0; b < a->num_blocks; ++b) {
    if (a->ref[b] < 0) return err(VALUE_ERROR, "negative reference count of block %d", b);
    if ((a->ref[b] == 0) != (seen[b] != 0)) return err(VALUE_ERROR, "free stack disagrees with reference count of block %d", b);
  }
  return OK;
}

// ------------------------------------------------------------------ block table
MS_EXPORT void* ms_table_create(void* alloc) { return new Table{static_cast<Allocator*>(alloc)}; }
MS_EXPORT void ms_table_destroy(void* h) { delete static_cast<Table*>(h); }
MS_EXPORT long long ms_table_num_tokens(void* h) { return static_cast<Table*>(h)->num_tokens; }
MS_EXPORT int ms_table_num_entries(void* h) { return (int)static_cast<Table*>(h)->blocks.size(); }
MS_EXPORT int ms_table_num_held(void* h) {
  auto* t = static_cast<Table*>(h);
  return (int)t->blocks.size() - t->first_live;
}

static int blocks_needed(const Table* t, long long n) {
  const long long bs = t->alloc->block_size;
  const long long want = (t->num_tokens + n + bs - 1) / bs;
  return (int)std::max<long long>(0, want - (long long)t->blocks.size());
}

MS_EXPORT int ms_table_blocks_needed(void* h, long long n, int* out) {
  if (n < 0) return err(VALUE_ERROR, "cannot append %lld tokens", n);
  *out = blocks_needed(static_cast<Table*>(h), n);
  return OK;
}

MS_EXPORT int ms_table_append_tokens(void* h, long long n) {
  auto* t = static_cast<Table*>(h);
  if (n < 0) return err(VALUE_ERROR, "cannot append %lld tokens", n);
  const int need = blocks_needed(t, n);
  const size_t old = t->blocks.size();
  t->blocks.resize(old + need);
  const int rc = ms_alloc_allocate(t->alloc, need, t->blocks.data() + old);
  if (rc != OK) {
    t->blocks.resize(old);
    return rc;
  }
  t->num_tokens += n;
  return OK;
}

MS_EXPORT int ms_table_slot(void* h, long long pos, long long* out) {
  auto* t = static_cast<Table*>(h);
  if (pos < 0 || pos >= t->num_tokens) return err(INDEX_ERROR, "position %lld out of range [0, %lld)", pos, t->num_tokens);
  const int bs = t->alloc->block_size;
  const int b = t->blocks[pos / bs];
  if (b < 0) return err(INDEX_ERROR, "position %lld lies in a page that was given back", pos);
  *out = (long long)b * bs + pos % bs;
  return OK;
}

MS_EXPORT int ms_table_rewind(void* h, long long n) {
  auto* t = static_cast<Table*>(h);
  if (n < 0 || n > t->num_tokens) return err(INDEX_ERROR, "cannot rewind %lld of %lld tokens", n, t->num_tokens);
  t->num_tokens -= n;
  return OK;
}

MS_EXPORT int ms_table_release(void* h) {
  auto* t = static_cast<Table*>(h);
  const int rc = ms_alloc_free(t->alloc, t->blocks.data() + t->first_live, (int)t->blocks.size() - t->first_live);
  if (rc != OK) return rc;
  t->blocks.clear();
  t->num_tokens = 0;
  t->first_live = 0;
  return OK;
}

// Give back every page that lies wholly below position `pos` (no later query looks that far
// back). Returns the number of pages freed in *freed.
MS_EXPORT int ms_table_release_below(void* h, long long pos, int* freed) {
  auto* t = static_cast<Table*>(h);
  const int bs = t->alloc->block_size;
  long long upto = std::min<long long>(std::max<long long>(pos, 0) / bs, (long long)t->blocks.size());
  // never the page that holds the newest token
  if (t->num_tokens > 0) upto = std::min<long long>(upto, (t->num_tokens - 1) / bs);
  *freed = 0;
  if (upto <= t->first_live) return OK;
  const int rc = ms_alloc_free(t->alloc, t->blocks.data() + t->first_live, (int)(upto - t->first_live));
  if (rc != OK) return rc;
  for (long long i = t->first_live; i < upto; ++i) t->blocks[i] = -1;
  *freed = (int)(upto - t->first_live);
  t->first_live = (int)upto;
  return OK;
}

MS_EXPORT int ms_table_copy_blocks(void* h, int* out, int cap) {
  auto* t = static_cast<Table*>(h);
  if ((int)t->blocks.size() > cap) return err(VALUE_ERROR, "buffer of %d entries for a table of %d", cap, (int)t->blocks.size());
  std::copy(t->blocks.begin(), t->blocks.end(), out);
  return OK;
}

// ------------------------------------------------------------------ step packer
// Arena layout (int32 entries; every field starts on a multiple of 4 entries):
//   token_ids[T'] positions[T'] row_of_token[T'] cu_q[R'+1] q_start[R'] kv_len[R'] state_slot[R']
//   logit_rows[W] then for each cache group g: page_indptr_g[R'+1] page_indices_g[P_g]
// with R' = rows + pad_rows and T' = tokens + pad_rows * pad_len. Of a table only the pages it still holds
// are packed (and the entry just below them, which reads -1): page_indptr_g[r] is the index that
// the table's entry 0 WOULD have, so that page_indices_g[page_indptr_g[r] + (position / page_size)]
// is right for every position a kernel may ask for (those the window still reaches), whatever a
// windowed group has given back; it can be negative. So a step never packs more entries than
// the pool has pages, plus one per row. A padding row is pad_len tokens 0 at
// positions 0 .. pad_len - 1 whose every page is `pad_page` (a page outside the allocator, of
// pad_page_size tokens; what the row's tokens write there overlaps and is never read for a result) and
// whose state slot is `pad_state_slot` (a slot no request gets, so that a mixer with state needs no
// mask); with want_pad_rows the logits of its last token are wanted too, so that the layout depends on R' alone. indices_cap > 0 gives every
// group's page_indices exactly that many entries (a layout that does not move with the number of
// pages, as a captured CUDA graph needs); 0 packs them tightly.
// offsets_out receives the start of each field: 8 + 2*groups entries, then the total.
static long long align4(long long x) { return (x + 3) & ~3LL; }

MS_EXPORT long long ms_pack_step(int32_t* arena, long long arena_cap, long long* offsets_out, int rows, int pad_rows,
                                 const int* q_start, const int* q_len, const int* token_ids,
                                 const int* state_slot, const int* logit_rows, int num_logit_rows, int groups,
                                 void* const* tables /* [groups][rows] */, const int* pad_page /* [groups] */,
                                 long long indices_cap, int want_pad_rows, int pad_state_slot, int pad_len,
                                 int pad_page_size) {
  if (rows < 0 || pad_rows < 0 || groups < 0) return -err(VALUE_ERROR, "pack_step: negative count");
  if (pad_len < 1 || pad_page_size < 1) return -err(VALUE_ERROR, "pack_step: a padding row of %d tokens on pages of %d", pad_len, pad_page_size);
  const long long pad_pages = (pad_len + pad_page_size - 1) / pad_page_size;
  long long T = 0;
  for (int r = 0; r < rows; ++r) {
    if (q_len[r] < 1) return -err(VALUE_ERROR, "pack_step: row %d brings %d tokens", r, q_len[r]);
    T += q_len[r];
  }
  const long long Tp = T + (long long)pad_rows * pad_len, Rp = rows + pad_rows;
  long long off = 0;
  int f = 0;
  auto field = [&](long long n) {
    offsets_out[f++] = off;
    const long long at = off;
    off = align4(off + n);
    return at;
  };
  const long long o_ids = field(Tp), o_pos = field(Tp), o_row = field(Tp), o_cu = field(Rp + 1), o_qs = field(Rp),
                  o_kv = field(Rp), o_ss = field(Rp), o_lr = field(num_logit_rows + (want_pad_rows ? pad_rows : 0));
  std::vector<long long> o_indptr(groups), o_indices(groups);
  for (int g = 0; g < groups; ++g) {
    long long pages = pad_rows * pad_pages;
    for (int r = 0; r < rows; ++r) {
      auto* t = static_cast<Table*>(tables[(size_t)g * rows + r]);
      if (t->num_tokens != (long long)q_start[r] + q_len[r])
        return -err(VALUE_ERROR, "pack_step: row %d, group %d: the table holds %lld tokens, the step ends at %d", r, g,
                    t->num_tokens, q_start[r] + q_len[r]);
      pages += (long long)t->blocks.size() - std::max(t->first_live - 1, 0);
    }
    if (indices_cap > 0 && pages > indices_cap)
      return -err(VALUE_ERROR, "pack_step: group %d needs %lld page entries, the fixed layout has %lld", g, pages, indices_cap);
    o_indptr[g] = field(Rp + 1);
    o_indices[g] = field(indices_cap > 0 ? indices_cap : pages);
  }
  offsets_out[f] = off;
  if (off > arena_cap) return -err(VALUE_ERROR, "pack_step: arena of %lld entries, step needs %lld", arena_cap, off);

  long long t = 0;
  arena[o_cu] = 0;
  for (int r = 0; r < Rp; ++r) {
    const bool pad = r >= rows;
    const int n = pad ? pad_len : q_len[r], s = pad ? 0 : q_start[r];
    for (int i = 0; i < n; ++i, ++t) {
      arena[o_ids + t] = pad ? 0 : token_ids[t];
      arena[o_pos + t] = s + i;
      arena[o_row + t] = r;
    }
    arena[o_cu + r + 1] = (int32_t)t;
    arena[o_qs + r] = s;
    arena[o_kv + r] = s + n;
    arena[o_ss + r] = pad ? pad_state_slot : (state_slot ? state_slot[r] : -1);
  }
  for (int i = 0; i < num_logit_rows; ++i) {
    if (logit_rows[i] < 0 || logit_rows[i] >= T) return -err(INDEX_ERROR, "pack_step: logit row %d outside [0, %lld)", logit_rows[i], T);
    arena[o_lr + i] = logit_rows[i];
  }
  if (want_pad_rows)
    for (int i = 0; i < pad_rows; ++i) arena[o_lr + num_logit_rows + i] = (int32_t)(T + (long long)(i + 1) * pad_len - 1);
  for (int g = 0; g < groups; ++g) {
    long long p = 0;
    for (int r = 0; r < Rp; ++r) {
      if (r < rows) {
        auto* tb = static_cast<Table*>(tables[(size_t)g * rows + r]);
        const int from = std::max(tb->first_live - 1, 0);
        arena[o_indptr[g] + r] = (int32_t)(p - from);
        std::copy(tb->blocks.begin() + from, tb->blocks.end(), arena + o_indices[g] + p);
        p += (long long)tb->blocks.size() - from;
      } else {
        arena[o_indptr[g] + r] = (int32_t)p;
        for (long long k = 0; k < pad_pages; ++k) arena[o_indices[g] + p++] = pad_page[g];
      }
    }
    arena[o_indptr[g] + Rp] = (int32_t)p;
  }
  return off;
}
