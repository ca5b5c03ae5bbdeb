// Host control plane: request scheduler + page (block) manager, plain host C++ behind a C ABI
// (include/zipage_b200_host.h).  Behaviour follows the reference's Python objects step for step
// (zipage/engine/scheduler.py, block_manager.py, sequence.py); the data layout does not: sequence
// and block state live in flat vectors, every queue (waiting, running, free blocks) is an
// intrusive doubly linked list over indices, so popleft / pop / append / appendleft / remove(x)
// are all O(1) (the reference's deque.remove is a linear search), and one call hands the runner
// the index arrays of a whole step.
#include <climits>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <mutex>
#include <unordered_map>
#include <vector>

#include "../../include/zipage_b200_host.h"

namespace zp {
namespace host {

static thread_local char g_err[256] = "";
static int fail(int code, const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
  return code;
}

// ---- XXH64 (seed 0), the published algorithm, one shot over a byte buffer --------------------
static inline uint64_t rotl64(uint64_t x, int r) { return (x << r) | (x >> (64 - r)); }
static inline uint64_t rd64(const unsigned char* p) { uint64_t v; memcpy(&v, p, 8); return v; }
static inline uint32_t rd32(const unsigned char* p) { uint32_t v; memcpy(&v, p, 4); return v; }
static const uint64_t XP1 = 11400714785074694791ull, XP2 = 14029467366897019727ull,
                      XP3 = 1609587929392839161ull, XP4 = 9650029242287828579ull,
                      XP5 = 2870177450012600261ull;
static inline uint64_t xround(uint64_t acc, uint64_t in) { return rotl64(acc + in * XP2, 31) * XP1; }
static inline uint64_t xmerge(uint64_t h, uint64_t v) { return (h ^ xround(0, v)) * XP1 + XP4; }
static uint64_t xxh64(const unsigned char* p, size_t len) {
  const unsigned char* end = p + len;
  uint64_t h;
  if (len >= 32) {
    uint64_t v1 = XP1 + XP2, v2 = XP2, v3 = 0, v4 = 0 - XP1;
    const unsigned char* limit = end - 32;
    do {
      v1 = xround(v1, rd64(p)); v2 = xround(v2, rd64(p + 8));
      v3 = xround(v3, rd64(p + 16)); v4 = xround(v4, rd64(p + 24));
      p += 32;
    } while (p <= limit);
    h = rotl64(v1, 1) + rotl64(v2, 7) + rotl64(v3, 12) + rotl64(v4, 18);
    h = xmerge(h, v1); h = xmerge(h, v2); h = xmerge(h, v3); h = xmerge(h, v4);
  } else {
    h = XP5;
  }
  h += (uint64_t)len;
  while (p + 8 <= end) { h ^= xround(0, rd64(p)); h = rotl64(h, 27) * XP1 + XP4; p += 8; }
  if (p + 4 <= end) { h ^= (uint64_t)rd32(p) * XP1; h = rotl64(h, 23) * XP2 + XP3; p += 4; }
  while (p < end) { h ^= (uint64_t)(*p) * XP5; h = rotl64(h, 11) * XP1; ++p; }
  h ^= h >> 33; h *= XP2; h ^= h >> 29; h *= XP3; h ^= h >> 32;
  return h;
}
// BlockManager.compute_hash: optional 8-byte little-endian prefix, then the tokens as int64
static uint64_t hash_tokens(const int32_t* tok, int n, bool has_prefix, uint64_t prefix) {
  std::vector<unsigned char> buf((size_t)n * 8 + (has_prefix ? 8 : 0));
  unsigned char* p = buf.data();
  if (has_prefix) { memcpy(p, &prefix, 8); p += 8; }
  for (int i = 0; i < n; ++i) { const int64_t v = tok[i]; memcpy(p, &v, 8); p += 8; }
  return xxh64(buf.data(), buf.size());
}

// ---- intrusive doubly linked list over indices ------------------------------------------------
struct Links { int32_t prev = -1, next = -1; };
struct List {
  int32_t head = -1, tail = -1, count = 0;
  template <typename V> void push_back(V& v, int i) {
    v[i].lk.prev = tail; v[i].lk.next = -1;
    if (tail >= 0) v[tail].lk.next = i; else head = i;
    tail = i; ++count;
  }
  template <typename V> void push_front(V& v, int i) {
    v[i].lk.next = head; v[i].lk.prev = -1;
    if (head >= 0) v[head].lk.prev = i; else tail = i;
    head = i; ++count;
  }
  template <typename V> void remove(V& v, int i) {
    const int p = v[i].lk.prev, n = v[i].lk.next;
    if (p >= 0) v[p].lk.next = n; else head = n;
    if (n >= 0) v[n].lk.prev = p; else tail = p;
    v[i].lk.prev = v[i].lk.next = -1; --count;
  }
  template <typename V> int pop_front(V& v) { const int i = head; remove(v, i); return i; }
  template <typename V> int pop_back(V& v) { const int i = tail; remove(v, i); return i; }
};

struct Seq {
  Links lk;
  std::vector<int32_t> tokens, table, new_table, to_release;
  int32_t num_tokens = 0, num_prompt = 0, num_cached = 0, last_token = 0, query_id = -1, max_tokens = 0;
  float temperature = 1.f;
  double time_prefilled = 0, time_finished = 0;
  uint8_t status = ZP_SEQ_WAITING, require_compress = 0, compressed = 0, prefilled = 0, ignore_eos = 0;
  uint8_t where = 0;   // which queue links it: 0 none, 1 waiting, 2 running
};

struct Block {
  Links lk;                 // position in the free list while free
  int32_t ref = 0;
  bool has_hash = false, is_free = true;
  uint64_t hash = 0;
  std::vector<int32_t> tokens;   // the tokens the hash was taken of (guards against collisions)
  void reset() { ref = 1; has_hash = false; hash = 0; tokens.clear(); }
};

struct Sched {
  zp_sched_config cfg;
  std::vector<Seq> seqs;
  std::vector<Block> blocks;
  List waiting, running, free_blocks;
  int32_t used_blocks = 0;
  std::deque<int32_t> free_qids;
  int32_t used_qids = 0;
  std::unordered_map<uint64_t, int32_t> hash_to_block;
  std::vector<int32_t> last_finished;   // handles that finished in the latest postprocess call
  // The reference engine's asynchronous mode calls postprocess() from its compression thread
  // while the main thread schedules (zipage_engine.py:88-96, :137-186); Python's interpreter lock
  // serialises its own objects, a foreign call releases that lock, so every entry point locks here.
  std::mutex mu;

  // ---- Sequence properties (sequence.py:62-76) ----
  int num_blocks(const Seq& s) const { return (s.num_tokens + cfg.block_size - 1) / cfg.block_size; }
  int last_block_num_tokens(const Seq& s) const { return s.num_tokens - (num_blocks(s) - 1) * cfg.block_size; }

  // ---- BlockManager ----
  // Block.reset (block_manager.py:20-23).  The reference leaves the block's old hash in
  // hash_to_block_id for ever; a later lookup that finds it compares token lists and misses.  Here
  // the entry is dropped (when it still points at this block), which gives the same misses and
  // keeps the map no larger than the number of blocks.
  void reset_block(int id) {
    Block& b = blocks[id];
    if (b.has_hash) {
      auto it = hash_to_block.find(b.hash);
      if (it != hash_to_block.end() && it->second == id) hash_to_block.erase(it);
    }
    b.reset();
  }
  void allocate_block(int id) {            // block_manager.py:59-66
    free_blocks.remove(blocks, id);
    blocks[id].is_free = false;
    ++used_blocks;
    reset_block(id);
  }
  void deallocate_block(int id) {          // :68-74
    Block& b = blocks[id];
    if (--b.ref == 0) {
      --used_blocks;
      b.is_free = true;
      free_blocks.push_back(blocks, id);
    }
  }
  bool can_allocate(const Seq& s) const { return free_blocks.count >= num_blocks(s); }   // :76-77
  int allocate(Seq& s);
  void deallocate(Seq& s) {                // :119-123
    for (size_t i = s.table.size(); i-- > 0;) deallocate_block(s.table[i]);
    s.num_cached = 0; s.prefilled = 0; s.table.clear();
  }
  void deallocate_to_release(Seq& s) {     // :125-127
    for (size_t i = s.to_release.size(); i-- > 0;) deallocate_block(s.to_release[i]);
    s.to_release.clear();
  }
  int may_compress(Seq& s, bool* ok);
  int can_append_or_compress(Seq& s, bool* ok);
  bool can_append(const Seq& s) const {    // :192-193
    return free_blocks.count >= (s.num_tokens % cfg.block_size == 1 ? 1 : 0);
  }
  int may_append(Seq& s);

  // ---- Scheduler ----
  void allocate_qid(Seq& s) { s.query_id = free_qids.front(); free_qids.pop_front(); ++used_qids; }   // :35-38
  void deallocate_qid(Seq& s) {            // :40-44
    if (s.query_id != -1) { free_qids.push_back(s.query_id); --used_qids; s.query_id = -1; }
  }
  bool can_decode_without_qid(const Seq& s) const {   // :126-130
    if (num_blocks(s) < cfg.max_blocks_per_seq) return true;
    return last_block_num_tokens(s) <= cfg.block_size - cfg.query_cache_len;
  }
  int preempt_popped(int h);
  int schedule(int32_t* out, int cap, int32_t* is_prefill);
  int postprocess(const int32_t* hs, int n, const int32_t* toks, double now);
};

// ---- BlockManager ------------------------------------------------------------------------------
// allocate (block_manager.py:79-113): one block per 256 tokens of the sequence; with the prefix
// cache, full blocks are looked up by the chained hash of their tokens until the first miss.
int Sched::allocate(Seq& s) {
  if (!s.table.empty()) return fail(ZP_SCHED_ERR_STATE, "allocate: the sequence already has blocks");
  const int BS = cfg.block_size, nb = num_blocks(s);
  bool has_h = false, cache_miss = false;
  uint64_t h = 0;
  for (int i = 0; i < nb; ++i) {
    const int lo = i * BS, n = (lo + BS <= s.num_tokens ? BS : s.num_tokens - lo);
    const int32_t* tok = s.tokens.data() + lo;
    if (n == BS && cfg.enable_prefix_cache) { h = hash_tokens(tok, n, has_h, h); has_h = true; }
    else has_h = false;
    int id = -1;
    if (has_h) {
      auto it = hash_to_block.find(h);
      if (it != hash_to_block.end()) id = it->second;
    }
    const bool may_save_query = (i == nb - 1 && nb >= cfg.max_blocks_per_seq);
    if (id == -1 || may_save_query || (int)blocks[id].tokens.size() != n ||
        memcmp(blocks[id].tokens.data(), tok, sizeof(int32_t) * n) != 0)
      cache_miss = true;
    if (cache_miss) {
      id = free_blocks.head;
      if (id < 0) return fail(ZP_SCHED_ERR_STATE, "allocate: no free block");
      allocate_block(id);
    } else {
      s.num_cached += BS;
      if (!blocks[id].is_free) ++blocks[id].ref;
      else allocate_block(id);
    }
    if (has_h) {
      blocks[id].has_hash = true; blocks[id].hash = h;
      blocks[id].tokens.assign(tok, tok + n);
      hash_to_block[h] = id;
    }
    s.table.push_back(id);
  }
  return 0;
}

// may_compress (block_manager.py:129-171): choose the destination pages of a compression.  A
// sequence compressed before keeps its first max_blocks_per_seq pages; a first compression must
// not write into pages shared through the prefix cache, so it takes fresh pages for those.
int Sched::may_compress(Seq& s, bool* ok) {
  const int MB = cfg.max_blocks_per_seq, n = (int)s.table.size();
  if (s.compressed) {
    const int keep = n < MB ? n : MB;
    s.new_table.assign(s.table.begin(), s.table.begin() + keep);
    s.to_release.assign(s.table.begin() + keep, s.table.end());
    s.require_compress = 1;
    *ok = true;
    return 0;
  }
  int nps = 0;   // leading pages that other sequences share
  while (nps < n && blocks[s.table[nps]].ref > 1) ++nps;
  if (n - nps < 1) return fail(ZP_SCHED_ERR_STATE, "may_compress: every page of the sequence is shared");
  const int num_new = nps < MB - 1 ? nps : MB - 1;
  if (num_new > free_blocks.count) { *ok = false; return 0; }
  s.new_table.clear();
  for (int i = 0; i < num_new; ++i) {
    const int id = free_blocks.head;
    allocate_block(id);
    s.new_table.push_back(id);
  }
  const int lo = nps, hi = (nps + MB - num_new < n) ? nps + MB - num_new : n;
  s.new_table.insert(s.new_table.end(), s.table.begin() + lo, s.table.begin() + hi);
  if ((int)s.new_table.size() != MB)
    return fail(ZP_SCHED_ERR_STATE, "may_compress: %d destination pages, expected %d", (int)s.new_table.size(), MB);
  s.to_release.assign(s.table.begin(), s.table.begin() + nps);
  s.to_release.insert(s.to_release.end(), s.table.begin() + hi, s.table.end());
  for (int i = lo; i < hi; ++i) reset_block(s.table[i]);
  s.require_compress = 1;
  *ok = true;
  return 0;
}

// can_append_or_compress (block_manager.py:173-190)
int Sched::can_append_or_compress(Seq& s, bool* ok) {
  *ok = true;
  if (s.require_compress) return 0;   // an asynchronous compression has not finished: skip this one
  const int BS = cfg.block_size, n = (int)s.table.size();
  if (s.num_tokens % BS == 1 && s.num_cached > BS * n) {
    if (n < cfg.max_blocks_per_seq) { if (free_blocks.count <= 0) *ok = false; }
    else return may_compress(s, ok);
  }
  return 0;
}

// may_append (block_manager.py:195-210)
int Sched::may_append(Seq& s) {
  if (s.require_compress) return 0;
  if (s.table.empty()) return fail(ZP_SCHED_ERR_STATE, "may_append: the sequence has no blocks");
  const int BS = cfg.block_size;
  Block& last = blocks[s.table.back()];
  if (s.num_tokens % BS == 1 && s.num_cached > BS * (int)s.table.size()) {
    const int id = free_blocks.head;
    if (id < 0) return fail(ZP_SCHED_ERR_STATE, "may_append: no free block");
    allocate_block(id);
    s.table.push_back(id);
  } else if (s.num_tokens % BS == 0) {
    if (!s.compressed) {
      const int nb = num_blocks(s);
      const int32_t* tok = s.tokens.data() + (size_t)(nb - 1) * BS;
      bool has_prefix = false;
      uint64_t prefix = 0;
      if (s.table.size() > 1) {
        const Block& before = blocks[s.table[s.table.size() - 2]];
        has_prefix = before.has_hash; prefix = before.hash;
      }
      const uint64_t h = hash_tokens(tok, BS, has_prefix, prefix);
      last.has_hash = true; last.hash = h;
      last.tokens.assign(tok, tok + BS);
      hash_to_block[h] = s.table.back();
    }
  } else if (last.has_hash) {
    return fail(ZP_SCHED_ERR_STATE, "may_append: the last block is hashed but not full");
  }
  return 0;
}

// ---- Scheduler -----------------------------------------------------------------------------------
// preempt (scheduler.py:136-141) of a sequence that has just been taken off the running queue
int Sched::preempt_popped(int h) {
  Seq& s = seqs[h];
  if (s.compressed || s.require_compress)
    return fail(ZP_SCHED_ERR_STATE, "preempt: sequence %d is compressed or waits for its compression", h);
  s.status = ZP_SEQ_WAITING;
  deallocate_qid(s);
  deallocate(s);
  waiting.push_front(seqs, h);
  s.where = 1;
  return 0;
}

// schedule (scheduler.py:47-124)
int Sched::schedule(int32_t* out, int cap, int32_t* is_prefill) {
  if (cap < cfg.max_num_seqs) return fail(ZP_SCHED_ERR_ARG, "schedule: room for %d handles, max_num_seqs is %d", cap, cfg.max_num_seqs);
  std::vector<int> keep, rejoin;
  // hybrid engine: sequences that run without an observation window get a slot when one is free
  if (cfg.enable_hybrid_engine && running.count && seqs[running.tail].query_id == -1) {
    while (running.count && !free_qids.empty()) {
      const int h = running.pop_front(seqs);
      keep.push_back(h);
      if (seqs[h].query_id == -1) allocate_qid(seqs[h]);
    }
    for (size_t i = keep.size(); i-- > 0;) running.push_front(seqs, keep[i]);
    keep.clear();
  }
  // prefill: admit waiting sequences while tokens, blocks and query slots last
  int n_out = 0, batched = 0;
  while (waiting.count && n_out < cfg.max_num_seqs) {
    const int h = waiting.head;
    Seq& s = seqs[h];
    if (batched + s.num_tokens > cfg.max_num_batched_tokens || !can_allocate(s)) break;
    if (free_qids.empty()) {
      if (!cfg.enable_hybrid_engine) break;
      if (!can_decode_without_qid(s)) break;
    }
    if (!free_qids.empty()) allocate_qid(s);
    const int rc = allocate(s);
    if (rc < 0) return rc;
    s.status = ZP_SEQ_RUNNING;
    waiting.pop_front(seqs);
    running.push_back(seqs, h);
    s.where = 2;
    if (s.num_cached != s.num_tokens) {
      batched += s.num_tokens - s.num_cached;
      out[n_out++] = h;
    }
  }
  if (n_out) { *is_prefill = 1; return n_out; }

  // decode: walk the running queue from the front; a sequence that cannot get the block it needs
  // makes room by preempting (or, if that one is compressed, setting aside) sequences at the back
  while (running.count && n_out < cfg.max_num_seqs) {
    const int h = running.pop_front(seqs);
    Seq& s = seqs[h];
    s.where = 0;
    rejoin.clear();
    if (s.query_id != -1) {
      for (;;) {
        bool ok;
        int rc = can_append_or_compress(s, &ok);
        if (rc < 0) return rc;
        if (ok) {
          rc = may_append(s);
          if (rc < 0) return rc;
          keep.push_back(h);
          out[n_out++] = h;
          break;
        }
        if (running.count && (seqs[running.tail].query_id == -1 || cfg.enable_prefix_cache)) {
          const int last = running.pop_back(seqs);
          seqs[last].where = 0;
          if (!(seqs[last].compressed || seqs[last].require_compress)) {
            rc = preempt_popped(last);
            if (rc < 0) return rc;
          } else {
            rejoin.push_back(last);
          }
        } else {
          keep.push_back(h);   // suspended without preemption
          break;
        }
      }
    } else {
      const bool not_blocking = can_decode_without_qid(s);
      for (;;) {
        if (!(not_blocking && !can_append(s))) {
          keep.push_back(h);
          if (not_blocking) {
            const int rc = may_append(s);
            if (rc < 0) return rc;
            out[n_out++] = h;
          }
          break;
        }
        if (running.count) {
          const int last = running.pop_back(seqs);
          seqs[last].where = 0;
          const int rc = preempt_popped(last);
          if (rc < 0) return rc;
        } else {
          keep.push_back(h);
          break;
        }
      }
    }
    for (size_t i = rejoin.size(); i-- > 0;) { running.push_back(seqs, rejoin[i]); seqs[rejoin[i]].where = 2; }
  }
  for (size_t i = keep.size(); i-- > 0;) { running.push_front(seqs, keep[i]); seqs[keep[i]].where = 2; }
  *is_prefill = 0;
  return n_out;
}

// postprocess (scheduler.py:143-167)
int Sched::postprocess(const int32_t* hs, int n, const int32_t* toks, double now) {
  const int BS = cfg.block_size;
  last_finished.clear();
  for (int i = 0; i < n; ++i) {
    const int h = hs[i];
    if (h < 0 || h >= (int)seqs.size()) return fail(ZP_SCHED_ERR_ARG, "postprocess: bad handle %d", h);
    Seq& s = seqs[h];
    if (s.require_compress) {     // the compression ran: its destination pages are the table now
      deallocate_to_release(s);
      s.table.swap(s.new_table);
      s.new_table.clear();
      s.num_cached = ((int)s.table.size() - 1) * BS + 1;
      s.compressed = 1;
      s.require_compress = 0;
    }
    if (toks) {
      const int32_t t = toks[i];
      s.tokens.push_back(t);      // Sequence.append_token (sequence.py:83-90)
      s.last_token = t;
      ++s.num_tokens;
      ++s.num_cached;
      s.prefilled = 1;
      const int done = s.num_tokens - s.num_prompt;
      if (done == 1) s.time_prefilled = now;
      if ((!s.ignore_eos && t == cfg.eos) || done == s.max_tokens) {
        s.time_finished = now;
        s.status = ZP_SEQ_FINISHED;
        deallocate(s);
        if (s.where != 2) return fail(ZP_SCHED_ERR_STATE, "postprocess: finished sequence %d is not running", h);
        running.remove(seqs, h);
        s.where = 0;
        deallocate_qid(s);
        last_finished.push_back(h);
      }
    }
  }
  return (int)last_finished.size();
}

}  // namespace host
}  // namespace zp

// ---- C ABI ---------------------------------------------------------------------------------------
using zp::host::Sched;
using zp::host::Seq;
using zp::host::fail;

static Sched* S(void* p) { return static_cast<Sched*>(p); }
static bool bad_handle(const Sched* s, int h) { return h < 0 || h >= (int)s->seqs.size(); }
static int copy_out(const std::vector<int32_t>& v, int32_t* out, int capacity) {
  if (out && capacity >= (int)v.size() && !v.empty()) memcpy(out, v.data(), sizeof(int32_t) * v.size());
  return (int)v.size();
}

static void seq_info_unlocked(const Seq& q, int32_t* out) {
  const int32_t v[16] = {q.status, q.num_tokens, q.num_prompt, q.num_cached, q.last_token, q.query_id,
                         q.require_compress, q.compressed, q.prefilled, q.max_tokens, q.ignore_eos,
                         (int32_t)q.table.size(), (int32_t)q.new_table.size(), (int32_t)q.to_release.size(), 0, 0};
  memcpy(out, v, sizeof(v));
}

extern "C" {

const char* zp_sched_last_error(void) { return zp::host::g_err; }

void* zp_sched_create(const zp_sched_config* cfg) {
  if (!cfg) { fail(ZP_SCHED_ERR_ARG, "zp_sched_create: null config"); return nullptr; }
  if (cfg->num_blocks < 1 || cfg->block_size < 1 || cfg->max_blocks_per_seq < 2 || cfg->max_num_seqs < 1 ||
      cfg->max_concurrency < 0 || cfg->query_cache_len < 0 || cfg->query_cache_len > cfg->block_size) {
    fail(ZP_SCHED_ERR_ARG, "zp_sched_create: bad configuration");
    return nullptr;
  }
  Sched* s = new Sched();
  s->cfg = *cfg;
  s->blocks.resize(cfg->num_blocks);
  for (int i = 0; i < cfg->num_blocks; ++i) s->free_blocks.push_back(s->blocks, i);
  for (int i = 0; i < cfg->max_concurrency; ++i) s->free_qids.push_back(i);
  return s;
}

void zp_sched_destroy(void* sched) { delete S(sched); }

int zp_sched_add(void* sched, const int32_t* token_ids, int n_tokens, float temperature, int max_tokens,
                 int ignore_eos) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !token_ids || n_tokens < 1) return fail(ZP_SCHED_ERR_ARG, "zp_sched_add: null argument or empty prompt");
  Sched* s = S(sched);
  s->seqs.emplace_back();
  const int h = (int)s->seqs.size() - 1;
  Seq& q = s->seqs[h];
  q.tokens.assign(token_ids, token_ids + n_tokens);
  q.num_tokens = q.num_prompt = n_tokens;
  q.last_token = token_ids[n_tokens - 1];
  q.temperature = temperature;
  q.max_tokens = max_tokens;
  q.ignore_eos = ignore_eos ? 1 : 0;
  s->waiting.push_back(s->seqs, h);
  q.where = 1;
  return h;
}

int zp_sched_schedule(void* sched, int32_t* out_handles, int capacity, int32_t* is_prefill) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !out_handles || !is_prefill) return fail(ZP_SCHED_ERR_ARG, "zp_sched_schedule: null argument");
  return S(sched)->schedule(out_handles, capacity, is_prefill);
}

int zp_sched_postprocess(void* sched, const int32_t* handles, int n, const int32_t* token_ids, double now,
                         int32_t* finished_out) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && !handles)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_postprocess: null argument");
  const int done = S(sched)->postprocess(handles, n, token_ids, now);
  if (done > 0 && finished_out) memcpy(finished_out, S(sched)->last_finished.data(), sizeof(int32_t) * done);
  return done;
}

int zp_sched_preempt(void* sched, int handle) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || bad_handle(S(sched), handle)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_preempt: bad handle");
  Sched* s = S(sched);
  Seq& q = s->seqs[handle];
  if (q.where == 1) return fail(ZP_SCHED_ERR_STATE, "zp_sched_preempt: sequence %d is already waiting", handle);
  if (q.compressed || q.require_compress) return s->preempt_popped(handle);   // reports the state error
  if (q.where == 2) { s->running.remove(s->seqs, handle); q.where = 0; }
  return s->preempt_popped(handle);
}

int zp_sched_mark_prefilled(void* sched, const int32_t* handles, int n) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && !handles)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_mark_prefilled: null argument");
  Sched* s = S(sched);
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_mark_prefilled: bad handle %d", handles[i]);
    s->seqs[handles[i]].num_cached = s->seqs[handles[i]].num_tokens;
  }
  return 0;
}

int zp_sched_release(void* sched, int handle) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || bad_handle(S(sched), handle)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_release: bad handle");
  Seq& q = S(sched)->seqs[handle];
  if (q.status != ZP_SEQ_FINISHED) return fail(ZP_SCHED_ERR_STATE, "zp_sched_release: sequence %d is not finished", handle);
  std::vector<int32_t>().swap(q.tokens);
  return 0;
}

int zp_sched_counts(void* sched, int32_t out[8]) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !out) return fail(ZP_SCHED_ERR_ARG, "zp_sched_counts: null argument");
  const Sched* s = S(sched);
  out[0] = s->waiting.count; out[1] = s->running.count;
  out[2] = s->free_blocks.count; out[3] = s->used_blocks;
  out[4] = (int32_t)s->free_qids.size(); out[5] = s->used_qids;
  out[6] = (int32_t)s->seqs.size();
  out[7] = (s->waiting.count == 0 && s->running.count == 0) ? 1 : 0;
  return 0;
}

int zp_sched_seq_info(void* sched, int handle, int32_t out[16]) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !out || bad_handle(S(sched), handle)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_info: bad argument");
  seq_info_unlocked(S(sched)->seqs[handle], out);
  return 0;
}

int zp_sched_seq_info_batch(void* sched, const int32_t* handles, int n, int32_t* out) {
  if (!sched || (n > 0 && (!handles || !out))) return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_info_batch: null argument");
  std::unique_lock<std::mutex> lock_(S(sched)->mu);
  for (int i = 0; i < n; ++i) {
    if (bad_handle(S(sched), handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_info_batch: bad handle %d", handles[i]);
    seq_info_unlocked(S(sched)->seqs[handles[i]], out + (size_t)i * 16);
  }
  return 0;
}

int zp_sched_seq_times(void* sched, int handle, double times[2], float* temperature) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !times || bad_handle(S(sched), handle)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_times: bad argument");
  const Seq& q = S(sched)->seqs[handle];
  times[0] = q.time_prefilled; times[1] = q.time_finished;
  if (temperature) *temperature = q.temperature;
  return 0;
}

int zp_sched_seq_set_num_cached(void* sched, int handle, int num_cached_tokens) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || bad_handle(S(sched), handle)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_set_num_cached: bad handle");
  S(sched)->seqs[handle].num_cached = num_cached_tokens;
  return 0;
}

int zp_sched_seq_list(void* sched, int handle, int which, int32_t* out, int capacity) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || bad_handle(S(sched), handle) || which < 0 || which > 3)
    return fail(ZP_SCHED_ERR_ARG, "zp_sched_seq_list: bad argument");
  const Seq& q = S(sched)->seqs[handle];
  return copy_out(which == 0 ? q.table : which == 1 ? q.new_table : which == 2 ? q.to_release : q.tokens, out, capacity);
}

int zp_sched_queue(void* sched, int which, int32_t* out, int capacity) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || which < 0 || which > 3) return fail(ZP_SCHED_ERR_ARG, "zp_sched_queue: bad argument");
  const Sched* s = S(sched);
  if (which == 3) {
    const int n = (int)s->free_qids.size();
    if (out && capacity >= n) for (int i = 0; i < n; ++i) out[i] = s->free_qids[i];
    return n;
  }
  const zp::host::List& l = which == 0 ? s->waiting : which == 1 ? s->running : s->free_blocks;
  if (out && capacity >= l.count) {
    int k = 0;
    if (which == 2) for (int i = l.head; i >= 0; i = s->blocks[i].lk.next) out[k++] = i;
    else for (int i = l.head; i >= 0; i = s->seqs[i].lk.next) out[k++] = i;
  }
  return l.count;
}

int zp_sched_block_info(void* sched, int block_id, int32_t out[2], uint64_t* hash) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !out || block_id < 0 || block_id >= (int)S(sched)->blocks.size())
    return fail(ZP_SCHED_ERR_ARG, "zp_sched_block_info: bad argument");
  const zp::host::Block& b = S(sched)->blocks[block_id];
  out[0] = b.ref; out[1] = b.has_hash ? 1 : 0;
  if (hash) *hash = b.hash;
  return 0;
}

uint64_t zp_sched_hash_tokens(const int32_t* token_ids, int n, int has_prefix, uint64_t prefix) {
  if (!token_ids || n < 0) return 0;
  return zp::host::hash_tokens(token_ids, n, has_prefix != 0, prefix);
}

int zp_sched_decode_inputs(void* sched, const int32_t* handles, int n, int32_t* input_ids,
                           int32_t* num_tokens, int32_t* query_ids, int32_t* block_tables, int table_width) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && (!handles || !input_ids || !num_tokens || !query_ids || !block_tables)))
    return fail(ZP_SCHED_ERR_ARG, "zp_sched_decode_inputs: null argument");
  const Sched* s = S(sched);
  int widest = 0;
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_decode_inputs: bad handle %d", handles[i]);
    const Seq& q = s->seqs[handles[i]];
    const int len = (int)q.table.size();
    if (len > table_width) return fail(ZP_SCHED_ERR_ARG, "zp_sched_decode_inputs: a table of %d blocks, %d columns", len, table_width);
    if (len > widest) widest = len;
    input_ids[i] = q.last_token;
    num_tokens[i] = q.num_tokens;
    query_ids[i] = q.query_id;
    int32_t* row = block_tables + (size_t)i * table_width;
    for (int j = 0; j < len; ++j) row[j] = q.table[j];
    for (int j = len; j < table_width; ++j) row[j] = -1;
  }
  return widest;
}

// number of window rows a prefill of `seqlen_q` new tokens stores (model_runner.py:328-339)
static int prefill_window_rows(const Sched* s, const Seq& q, int seqlen_q, int* start) {
  const int BS = s->cfg.block_size, QCL = s->cfg.query_cache_len;
  if (q.query_id == -1 || seqlen_q <= 0) return 0;
  const int nb = (seqlen_q + BS - 1) / BS;
  const int last = seqlen_q - (nb - 1) * BS;
  if (last <= BS - QCL) return 0;
  *start = nb * BS - QCL;
  return seqlen_q - *start;
}

int zp_sched_prefill_sizes(void* sched, const int32_t* handles, int n, int32_t out[4]) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || !out || (n > 0 && !handles)) return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_sizes: null argument");
  const Sched* s = S(sched);
  int64_t tokens = 0, rows = 0;
  int maxq = 0, maxk = 0;
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_sizes: bad handle %d", handles[i]);
    const Seq& q = s->seqs[handles[i]];
    const int lq = q.num_tokens - q.num_cached;
    int start = 0;
    tokens += lq;
    rows += prefill_window_rows(s, q, lq, &start);
    if (lq > maxq) maxq = lq;
    if (q.num_tokens > maxk) maxk = q.num_tokens;
  }
  if (tokens > INT32_MAX) return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_sizes: more than 2^31 tokens");
  out[0] = (int32_t)tokens; out[1] = (int32_t)rows; out[2] = maxq; out[3] = maxk;
  return 0;
}

int zp_sched_prefill_inputs(void* sched, const int32_t* handles, int n, int32_t* input_ids, int32_t* positions,
                            int32_t* slot_mapping, int32_t* cu_seqlens_q, int32_t* cu_seqlens_k,
                            int32_t* query_triples) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && (!handles || !input_ids || !positions || !slot_mapping || !cu_seqlens_q || !cu_seqlens_k)))
    return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_inputs: null argument");
  Sched* s = S(sched);
  const int BS = s->cfg.block_size;
  int64_t t = 0, rows = 0;
  if (n > 0) { cu_seqlens_q[0] = 0; cu_seqlens_k[0] = 0; }
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_inputs: bad handle %d", handles[i]);
    Seq& q = s->seqs[handles[i]];
    const int len = q.num_tokens, cached = q.num_cached, lq = len - cached;
    if (lq < 0 || (int)q.tokens.size() < len)
      return fail(ZP_SCHED_ERR_STATE, "zp_sched_prefill_inputs: sequence %d holds %d tokens, %d cached", handles[i], len, cached);
    int start = 0;
    const int wr = prefill_window_rows(s, q, lq, &start);
    if (wr > 0 && !query_triples) return fail(ZP_SCHED_ERR_ARG, "zp_sched_prefill_inputs: window rows but no triple array");
    for (int k = 0; k < wr; ++k) {
      int32_t* tr = query_triples + (rows + k) * 3;
      tr[0] = (int32_t)(t + start + k); tr[1] = q.query_id; tr[2] = k;
    }
    rows += wr;
    for (int k = 0; k < lq; ++k) { input_ids[t + k] = q.tokens[cached + k]; positions[t + k] = cached + k; }
    // slots of the blocks that are not cached yet (model_runner.py:379-386)
    const int nb = s->num_blocks(q), last = s->last_block_num_tokens(q);
    if (!q.table.empty()) {
      if ((int)q.table.size() < nb) return fail(ZP_SCHED_ERR_STATE, "zp_sched_prefill_inputs: sequence %d has %d blocks, needs %d", handles[i], (int)q.table.size(), nb);
      int64_t w = t;
      for (int b = cached / BS; b < nb; ++b) {
        const int cnt = (b != nb - 1) ? BS : last;
        const int32_t base = q.table[b] * BS;
        for (int k = 0; k < cnt; ++k) slot_mapping[w++] = base + k;
      }
      if (w - t != lq) return fail(ZP_SCHED_ERR_STATE, "zp_sched_prefill_inputs: sequence %d: %d slots for %d tokens (cached tokens must be whole blocks)", handles[i], (int)(w - t), lq);
      q.num_cached = len;          // model_runner.py:387
    }
    t += lq;
    cu_seqlens_q[i + 1] = (int32_t)t;
    cu_seqlens_k[i + 1] = cu_seqlens_k[i] + len;
  }
  return (int)rows;
}

int zp_sched_temperatures(void* sched, const int32_t* handles, int n, float* out) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && (!handles || !out))) return fail(ZP_SCHED_ERR_ARG, "zp_sched_temperatures: null argument");
  const Sched* s = S(sched);
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_temperatures: bad handle %d", handles[i]);
    out[i] = s->seqs[handles[i]].temperature;
  }
  return 0;
}

int zp_sched_compress_due(void* sched, const int32_t* handles, int n, int32_t* out_handles) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && (!handles || !out_handles))) return fail(ZP_SCHED_ERR_ARG, "zp_sched_compress_due: null argument");
  const Sched* s = S(sched);
  int k = 0;
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_compress_due: bad handle %d", handles[i]);
    if (s->seqs[handles[i]].require_compress) out_handles[k++] = handles[i];
  }
  return k;
}

int zp_sched_compress_inputs(void* sched, const int32_t* handles, int n, int32_t* tables, int table_width,
                             int32_t* targets, int target_width, int32_t* query_ids, uint8_t* compressed) {
  std::unique_lock<std::mutex> lock_;
  if (sched) lock_ = std::unique_lock<std::mutex>(S(sched)->mu);
  if (!sched || (n > 0 && (!handles || !tables || !targets || !query_ids || !compressed)))
    return fail(ZP_SCHED_ERR_ARG, "zp_sched_compress_inputs: null argument");
  const Sched* s = S(sched);
  int widest = 0;
  for (int i = 0; i < n; ++i) {
    if (bad_handle(s, handles[i])) return fail(ZP_SCHED_ERR_ARG, "zp_sched_compress_inputs: bad handle %d", handles[i]);
    const Seq& q = s->seqs[handles[i]];
    const int len = (int)q.table.size(), nt = (int)q.new_table.size();
    if (!q.require_compress || len < 1 || nt != target_width)
      return fail(ZP_SCHED_ERR_STATE, "zp_sched_compress_inputs: sequence %d is not due (%d blocks, %d destination pages)", handles[i], len, nt);
    if (len > table_width) return fail(ZP_SCHED_ERR_ARG, "zp_sched_compress_inputs: a table of %d blocks, %d columns", len, table_width);
    if (len > widest) widest = len;
    int32_t* row = tables + (size_t)i * table_width;
    for (int j = 0; j < len - 1; ++j) row[j] = q.table[j];
    row[len - 1] = -q.table[len - 1] - 2;     // the page that holds the observation window
    for (int j = len; j < table_width; ++j) row[j] = -1;
    memcpy(targets + (size_t)i * target_width, q.new_table.data(), sizeof(int32_t) * nt);
    query_ids[i] = q.query_id;
    compressed[i] = q.compressed;
  }
  return widest;
}

}  // extern "C"
