// Host-side bookkeeping of the inference engine: KV page allocation and the token queue.
//
// The reference keeps these structures on the accelerator and updates them with compiled scalar loops
// (src/levanter/inference/page_table.py:143-275, jit_scheduler.py:484-577).  Here they live in host memory: the scheduler
// runs on the CPU while the GPU executes the previous round, and each round ships one small PageBatchInfo to the device.
// All arrays are caller-owned int32 buffers (numpy), updated in place; the Python layer copies first where it wants
// value semantics.
#include <algorithm>
#include <cstdint>
#include <cstring>
#include <vector>

namespace {
constexpr int kInvalid = 2000000;
inline bool valid(int x) { return x >= 0 && x != kInvalid; }
}  // namespace

extern "C" {

// Allocate pages for the tokens (slot_ids[i], pos_ids[i]), i < n_tokens.  Tokens of one sequence must be contiguous.
// seq_lens[slot] becomes max(seq_lens[slot], max position + 1) for used slots; every page index needed to cover the new
// length is taken from the lowest-numbered free page.  Outputs describe the batch: one entry per distinct sequence in
// order of first appearance.
//   out_slot_ids[max_seqs], out_page_indices[max_seqs * pages_per_seq], out_seq_lens[max_seqs], out_cu_q_lens[max_seqs + 1],
//   out_token_dests[n_tokens] (page * page_size + offset, or INVALID), *out_num_seqs.
// Returns 0, or -5 when the table ran out of free pages (the table is left partially updated; callers treat it as fatal).
int lvb_pt_allocate(int* page_indices, int* ref_counts, int* seq_lens, const uint8_t* used, int max_seqs, int pages_per_seq,
                    int num_pages, int page_size, const int* slot_ids, const int* pos_ids, int n_tokens, int* out_slot_ids,
                    int* out_page_indices, int* out_seq_lens, int* out_cu_q_lens, int* out_num_seqs, int* out_token_dests) {
  std::fill(out_slot_ids, out_slot_ids + max_seqs, kInvalid);
  std::fill(out_page_indices, out_page_indices + static_cast<size_t>(max_seqs) * pages_per_seq, kInvalid);
  std::fill(out_seq_lens, out_seq_lens + max_seqs, kInvalid);
  std::fill(out_token_dests, out_token_dests + n_tokens, kInvalid);
  // group tokens by sequence in order of appearance
  int num = 0;
  std::vector<int> counts(max_seqs + 1, 0), max_pos(max_seqs + 1, -1);
  std::vector<int> dense_of_slot(max_seqs, -1);
  int pad_count = 0;
  for (int i = 0; i < n_tokens; ++i) {
    const int s = slot_ids[i];
    if (s < 0 || s >= max_seqs) { ++pad_count; continue; }
    int d = dense_of_slot[s];
    if (d < 0) {
      if (num >= max_seqs) continue;
      d = num++;
      dense_of_slot[s] = d;
      out_slot_ids[d] = s;
    }
    counts[d] += 1;
    if (valid(pos_ids[i])) max_pos[d] = std::max(max_pos[d], pos_ids[i]);
  }
  // cumulative query lengths over the dense sequences; padding tokens trail
  out_cu_q_lens[0] = 0;
  for (int d = 0; d < max_seqs; ++d) out_cu_q_lens[d + 1] = out_cu_q_lens[d] + (d < num ? counts[d] : (d == num ? pad_count : 0));
  int cursor = 0;
  for (int d = 0; d < num; ++d) {
    const int s = out_slot_ids[d];
    if (!used[s]) continue;
    const int old_len = seq_lens[s];
    const int new_len = std::max(old_len, max_pos[d] + 1);
    seq_lens[s] = new_len;
    const int old_pages = (old_len + page_size - 1) / page_size;
    const int new_pages = (new_len + page_size - 1) / page_size;
    for (int p = old_pages; p < new_pages && p < pages_per_seq; ++p) {
      while (cursor < num_pages && ref_counts[cursor] != 0) ++cursor;
      if (cursor >= num_pages) return -5;
      ref_counts[cursor] += 1;
      page_indices[static_cast<size_t>(s) * pages_per_seq + p] = cursor;
    }
  }
  for (int d = 0; d < num; ++d) {
    const int s = out_slot_ids[d];
    std::memcpy(out_page_indices + static_cast<size_t>(d) * pages_per_seq, page_indices + static_cast<size_t>(s) * pages_per_seq,
                sizeof(int) * pages_per_seq);
    out_seq_lens[d] = seq_lens[s];
  }
  *out_num_seqs = num;
  for (int i = 0; i < n_tokens; ++i) {
    const int s = slot_ids[i], pos = pos_ids[i];
    if (s < 0 || s >= max_seqs || !valid(pos)) continue;
    const int pi = pos / page_size;
    if (pi >= pages_per_seq) continue;
    const int page = page_indices[static_cast<size_t>(s) * pages_per_seq + pi];
    if (valid(page)) out_token_dests[i] = page * page_size + pos % page_size;
  }
  return 0;
}

// Release every page of the sequences with finished[s] != 0 and clear their slots.
void lvb_pt_free_finished(int* page_indices, int* ref_counts, int* seq_lens, uint8_t* used, int max_seqs, int pages_per_seq,
                          const uint8_t* finished) {
  for (int s = 0; s < max_seqs; ++s) {
    if (!finished[s]) continue;
    int* row = page_indices + static_cast<size_t>(s) * pages_per_seq;
    for (int p = 0; p < pages_per_seq; ++p) {
      if (valid(row[p])) ref_counts[row[p]] = std::max(ref_counts[row[p]] - 1, 0);
      row[p] = kInvalid;
    }
    seq_lens[s] = 0;
    used[s] = 0;
  }
}

// Make dst share src's full pages; a partial last page gets a fresh page for dst (the caller copies its contents).
// Returns the fresh page index, -1 if none was needed, or -5 when no page is free.
int lvb_pt_clone(int* page_indices, int* ref_counts, int* seq_lens, uint8_t* used, int pages_per_seq, int num_pages,
                 int page_size, int src, int dst) {
  const int* srow = page_indices + static_cast<size_t>(src) * pages_per_seq;
  int* drow = page_indices + static_cast<size_t>(dst) * pages_per_seq;
  const int len = seq_lens[src];
  const int used_pages = (len + page_size - 1) / page_size;
  const bool boundary = (len % page_size) == 0;
  std::memcpy(drow, srow, sizeof(int) * pages_per_seq);
  const int shared = used_pages - (boundary ? 0 : 1);
  for (int p = 0; p < shared; ++p)
    if (valid(srow[p])) ref_counts[srow[p]] += 1;
  int fresh = -1;
  if (!boundary) {
    int c = 0;
    while (c < num_pages && ref_counts[c] != 0) ++c;
    if (c >= num_pages) return -5;
    ref_counts[c] += 1;
    drow[std::max(used_pages - 1, 0)] = c;
    fresh = c;
  }
  seq_lens[dst] = len;
  used[dst] = 1;
  return fresh;
}

// Token queue: dequeue up to max_tokens entries, stable-sorted by slot id, into out_*; the remainder slides to the front.
// Returns the number of tokens dequeued.
int lvb_tq_pack_next(int* q_tokens, int* q_slots, int* q_pos, int* num_queued, int capacity, int max_tokens, int* out_tokens,
                     int* out_slots, int* out_pos) {
  const int n = std::min(*num_queued, max_tokens);
  std::vector<int> order(n);
  for (int i = 0; i < n; ++i) order[i] = i;
  std::stable_sort(order.begin(), order.end(), [&](int a, int b) { return q_slots[a] < q_slots[b]; });
  for (int i = 0; i < max_tokens; ++i) {
    if (i < n) {
      out_tokens[i] = q_tokens[order[i]];
      out_slots[i] = q_slots[order[i]];
      out_pos[i] = q_pos[order[i]];
    } else {
      out_tokens[i] = out_slots[i] = out_pos[i] = kInvalid;
    }
  }
  const int rest = *num_queued - n;
  std::memmove(q_tokens, q_tokens + n, sizeof(int) * rest);
  std::memmove(q_slots, q_slots + n, sizeof(int) * rest);
  std::memmove(q_pos, q_pos + n, sizeof(int) * rest);
  for (int i = rest; i < capacity; ++i) q_tokens[i] = q_slots[i] = q_pos[i] = kInvalid;
  *num_queued = rest;
  return n;
}

}  // extern "C"
