// Paged-KV block allocator: a free list of fixed-size blocks and one block table per sequence.
// Semantics follow the reference's PagedCache (crates/nn/src/kv_cache.rs:382-432) with its defect removed: a
// second reservation for a sequence extends the table instead of overwriting it (kv_cache.rs:420-423).
#include <mutex>
#include <unordered_map>
#include <vector>

#include "rb_runtime.h"

struct RbBlockAllocator {
  int num_blocks, block_size;
  std::vector<int32_t> free_list;                                // stack; lowest ids are handed out first
  std::unordered_map<int64_t, std::vector<int32_t>> tables;
  mutable std::mutex mu;
};

extern "C" {

RbBlockAllocator* rb_ba_create(int num_blocks, int block_size) {
  if (num_blocks <= 0 || block_size <= 0) return nullptr;
  auto* a = new RbBlockAllocator;
  a->num_blocks = num_blocks;
  a->block_size = block_size;
  a->free_list.reserve(num_blocks);
  for (int i = num_blocks - 1; i >= 0; --i) a->free_list.push_back(i);
  return a;
}
void rb_ba_destroy(RbBlockAllocator* a) { delete a; }
int rb_ba_num_free(const RbBlockAllocator* a) { std::lock_guard<std::mutex> l(a->mu); return (int)a->free_list.size(); }
int rb_ba_num_blocks(const RbBlockAllocator* a) { return a->num_blocks; }
int rb_ba_block_size(const RbBlockAllocator* a) { return a->block_size; }

static int blocks_for(const RbBlockAllocator* a, int tokens) { return (tokens + a->block_size - 1) / a->block_size; }

int rb_ba_can_reserve(const RbBlockAllocator* a, int64_t seq_id, int num_tokens) {
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  const int have = it == a->tables.end() ? 0 : (int)it->second.size();
  const int need = blocks_for(a, num_tokens) - have;
  return need <= (int)a->free_list.size() ? 1 : 0;
}

int rb_ba_reserve(RbBlockAllocator* a, int64_t seq_id, int num_tokens) {
  if (num_tokens < 0) return -1;
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  const int have = it == a->tables.end() ? 0 : (int)it->second.size();
  const int need = blocks_for(a, num_tokens) - have;
  if (need <= 0) {
    if (it == a->tables.end()) a->tables[seq_id];
    return 0;
  }
  if (need > (int)a->free_list.size()) return -1;
  auto& tab = a->tables[seq_id];
  for (int i = 0; i < need; ++i) {
    tab.push_back(a->free_list.back());
    a->free_list.pop_back();
  }
  return need;
}

int rb_ba_free(RbBlockAllocator* a, int64_t seq_id) {
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  if (it == a->tables.end()) return 0;
  const int n = (int)it->second.size();
  for (auto rit = it->second.rbegin(); rit != it->second.rend(); ++rit) a->free_list.push_back(*rit);
  a->tables.erase(it);
  return n;
}

int rb_ba_table_len(const RbBlockAllocator* a, int64_t seq_id) {
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  return it == a->tables.end() ? -1 : (int)it->second.size();
}

int rb_ba_table(const RbBlockAllocator* a, int64_t seq_id, int32_t* out, int max_out) {
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  if (it == a->tables.end()) return -1;
  const int n = (int)it->second.size();
  for (int i = 0; i < n && i < max_out; ++i) out[i] = it->second[i];
  return n;
}

int64_t rb_ba_slot(const RbBlockAllocator* a, int64_t seq_id, int token_index) {
  std::lock_guard<std::mutex> l(a->mu);
  auto it = a->tables.find(seq_id);
  if (it == a->tables.end() || token_index < 0) return -1;
  const int b = token_index / a->block_size;
  if (b >= (int)it->second.size()) return -1;
  return (int64_t)it->second[b] * a->block_size + token_index % a->block_size;
}

int rb_ba_num_sequences(const RbBlockAllocator* a) { std::lock_guard<std::mutex> l(a->mu); return (int)a->tables.size(); }

}  // extern "C"
