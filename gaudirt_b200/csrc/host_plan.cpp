// Host side of the C ABI: status text, pool geometry, paged-metadata validation and the
// length-aware split-KV schedule.  Nothing here touches the device.
#include "../../include/gaudirt_b200.h"

#include <algorithm>
#include <array>
#include <climits>
#include <functional>
#include <cstdint>
#include <numeric>
#include <string>
#include <unordered_map>
#include <vector>

namespace {
thread_local std::string g_metadata_error;

int metadata_fail(const char* message) {
  g_metadata_error = message;
  return GK_ERR_METADATA;
}

inline int64_t round_up(int64_t v, int64_t m) { return (v + m - 1) / m * m; }
}  // namespace

namespace gk {
extern thread_local int g_last_cuda_error;
}

extern "C" const char* gk_status_string(int status) {
  switch (status) {
    case GK_OK: return "ok";
    case GK_ERR_INVALID_ARGUMENT: return "invalid argument (null pointer, negative size, misaligned pointer or stride)";
    case GK_ERR_UNSUPPORTED: return "unsupported geometry";
    case GK_ERR_CUDA: return "CUDA launch failed";
    case GK_ERR_CAPACITY: return "output array or scratch area too small";
    case GK_ERR_METADATA: return "paged metadata rejected";
    default: return "unknown status";
  }
}

extern "C" int gk_abi_version(void) { return 1; }
extern "C" int gk_last_cuda_error(void) { return gk::g_last_cuda_error; }
extern "C" const char* gk_metadata_error(void) { return g_metadata_error.c_str(); }

extern "C" int gk_paged_kv_pool_bytes(int64_t layers, int64_t slots, int64_t kv_heads, int64_t head_dim,
                                      uint64_t* bytes_out) {
  if (!bytes_out) return GK_ERR_INVALID_ARGUMENT;
  // Geometry limits of allocate_paged_kv (src/bridge/paged_kv_pool.cpp:16-20) without its
  // 131072-slot descriptor cap; slots stay addressable by int32 slot ids.
  if (layers <= 0 || layers > 4096 || slots <= 0 || slots > INT32_MAX || kv_heads <= 0 || kv_heads > 256 ||
      (head_dim != 64 && head_dim != 128 && head_dim != 256))
    return GK_ERR_UNSUPPORTED;
  const uint64_t layer = 2ull * (uint64_t)slots * (uint64_t)kv_heads * (uint64_t)head_dim * 2ull;
  if (layer > UINT64_MAX / (uint64_t)layers) return GK_ERR_UNSUPPORTED;
  *bytes_out = layer * (uint64_t)layers;
  return GK_OK;
}

extern "C" int gk_paged_metadata_validate(const int32_t* locations, const int32_t* requests, const int32_t* positions,
                                          int64_t rows, const int32_t* mapping, int64_t n_requests, int64_t context,
                                          int64_t slots, int32_t* seq_out, int64_t* n_seq_out,
                                          int32_t* page_tokens_out) {
  if (!locations || !requests || !positions || !mapping || !seq_out || !n_seq_out) return GK_ERR_INVALID_ARGUMENT;
  if (rows <= 0 || rows > INT32_MAX || slots <= 0 || slots > INT32_MAX || n_requests <= 0 || n_requests > INT32_MAX ||
      context <= 0 || context > INT32_MAX || n_requests * context > INT32_MAX)
    return metadata_fail("GaudiRT: paged metadata dimensions outside supported range");
  const int64_t cells = n_requests * context;
  for (int64_t i = 0; i < cells; ++i)
    if (mapping[i] < -1 || mapping[i] >= slots) return metadata_fail("GaudiRT: request-to-token slot is out of range");

  std::vector<int32_t> reach(n_requests, -1);
  std::unordered_map<int32_t, std::pair<int32_t, int32_t>> target;   // output slot -> (request, position)
  target.reserve((size_t)rows * 2);
  // One bit per slot in front of the map: the prefix walk below touches every visible position,
  // almost none of which is an output slot of this step.
  std::vector<uint64_t> is_target(static_cast<size_t>(slots / 64 + 1), 0);
  int64_t n_seq = 0;
  for (int64_t i = 0; i < rows; ++i) {
    const int64_t slot = locations[i], request = requests[i], position = positions[i];
    if (slot < 0 || slot >= slots || request < 0 || request >= n_requests || position < 0 || position >= context)
      return metadata_fail("GaudiRT: paged metadata index is out of range");
    if (mapping[request * context + position] != slot)
      return metadata_fail("GaudiRT: output slot does not match request-to-token mapping");
    if (!target.emplace((int32_t)slot, std::make_pair((int32_t)request, (int32_t)position)).second)
      return metadata_fail("GaudiRT: duplicate output KV slot");
    is_target[static_cast<size_t>(slot >> 6)] |= 1ull << (slot & 63);
    const bool continues = i > 0 && requests[i - 1] == request && positions[i - 1] + 1 == position;
    if (continues) {
      ++seq_out[(n_seq - 1) * 4 + 1];
    } else {
      int32_t* s = seq_out + n_seq * 4;
      s[0] = (int32_t)i;
      s[1] = 1;
      s[2] = (int32_t)position;
      s[3] = (int32_t)request;
      ++n_seq;
    }
    reach[request] = std::max(reach[request], (int32_t)position);
  }
  int page = 128;
  for (int64_t request = 0; request < n_requests; ++request) {
    const int32_t* row = mapping + request * context;
    for (int32_t position = 0; position <= reach[request]; ++position) {
      const int32_t slot = row[position];
      if (slot < 0) return metadata_fail("GaudiRT: missing KV slot in a visible prefix");
      if (is_target[static_cast<size_t>(slot >> 6)] >> (slot & 63) & 1) {
        const auto hit = target.find(slot);
        if (hit != target.end() && (hit->second.first != request || hit->second.second != position))
          return metadata_fail("GaudiRT: output KV slot aliases another visible prefix position");
      }
      // A break in slot contiguity at `position` only allows pages that end there.
      if (position > 0 && slot != row[position - 1] + 1) page = std::min(page, position & -position);
    }
  }
  *n_seq_out = n_seq;
  if (page_tokens_out) *page_tokens_out = page;
  return GK_OK;
}

// Host half of slot allocation (src/bridge/paged_slot_allocator.cpp:95-128): the argument checks
// and one {prefix, length, first token, first fresh page} record per request.
extern "C" int gk_paged_slots_layout(const int64_t* prefixes, const int64_t* lengths, int64_t n_requests,
                                     int64_t page_size, int64_t free_page_count, int32_t* records_out,
                                     int64_t* total_out, int64_t* pages_out) {
  if (!prefixes || !lengths || !total_out || !pages_out) return GK_ERR_INVALID_ARGUMENT;
  if (page_size < 1 || page_size > INT32_MAX || n_requests <= 0 || n_requests > (int64_t{1} << 30))
    return metadata_fail("GaudiRT paged allocator: unsupported page size or request count");
  int64_t total = 0, pages = 0;
  for (int64_t i = 0; i < n_requests; ++i) {
    const int64_t prefix = prefixes[i], length = lengths[i];
    if (prefix < 0 || length < 0 || prefix > INT32_MAX || length > INT32_MAX || prefix + length > INT32_MAX)
      return metadata_fail("GaudiRT paged allocator: invalid request lengths");
    if (records_out && total <= INT32_MAX && pages <= INT32_MAX) {
      int32_t* r = records_out + i * 4;
      r[0] = (int32_t)prefix;
      r[1] = (int32_t)length;
      r[2] = (int32_t)total;
      r[3] = (int32_t)pages;
    }
    total += length;
    pages += (prefix + length + page_size - 1) / page_size - (prefix + page_size - 1) / page_size;
  }
  if (total <= 0 || total > (int64_t{1} << 30) || pages > (int64_t{1} << 30) || pages > free_page_count)
    return metadata_fail("GaudiRT paged allocator: invalid token count or insufficient free pages");
  *total_out = total;
  *pages_out = pages;
  return GK_OK;
}

extern "C" int gk_attention_plan_build(const int32_t* seq, int64_t n_seq, int q_heads, int kv_heads, int head_dim,
                                       int window, int sm_count, int split_tokens, int32_t* work_out,
                                       int64_t work_cap, int64_t* n_work_out, int32_t* combine_out,
                                       int64_t combine_cap, int64_t* n_combine_out, int64_t* partial_entries_out) {
  if (!seq || n_seq <= 0 || !n_work_out || !n_combine_out || !partial_entries_out || sm_count <= 0 ||
      split_tokens < 0 || (window != -1 && window <= 0))
    return GK_ERR_INVALID_ARGUMENT;
  if (q_heads <= 0 || q_heads > 256 || kv_heads <= 0 || kv_heads > 256 || q_heads % kv_heads != 0 ||
      (head_dim != 64 && head_dim != 128 && head_dim != 256) || q_heads / kv_heads > GK_MAX_PACKED_ROWS)
    return GK_ERR_UNSUPPORTED;
  const int group = q_heads / kv_heads;
  const int block_rows = std::max(1, GK_MAX_PACKED_ROWS / group);

  struct Block { int32_t first_row, n_rows, first_pos, table_row, lo, hi; };
  std::vector<Block> blocks;
  int64_t total_span = 0;
  for (int64_t s = 0; s < n_seq; ++s) {
    const int32_t* r = seq + s * 4;
    if (r[1] <= 0 || r[2] < 0 || r[0] < 0 || r[3] < 0) return GK_ERR_INVALID_ARGUMENT;
    for (int32_t done = 0; done < r[1]; done += block_rows) {
      const int32_t n = std::min<int32_t>(block_rows, r[1] - done);
      const int64_t first_pos = (int64_t)r[2] + done;
      if (first_pos + n > INT32_MAX) return GK_ERR_UNSUPPORTED;
      const int32_t lo = window > 0 ? (int32_t)std::max<int64_t>(0, first_pos - window + 1) : 0;
      blocks.push_back({r[0] + done, n, (int32_t)first_pos, r[3], lo, (int32_t)(first_pos + n)});
      total_span += blocks.back().hi - lo;
    }
  }
  // How a block's KV range is cut for a given longest-range limit.  Even cut: equal pieces, multiples
  // of the 64 tokens four warps eat, and no cut for ranges within 25 % of the limit.  Uneven cut: pieces
  // of exactly `chunk` tokens and the remainder as the last piece (a remainder under 64 tokens stays with
  // the piece before it).  The uneven cut is what fills the machine when a few hundred equal ranges meet
  // a slightly larger number of resident CTA slots: every range gives up its tail, and the tails fill
  // the slots that would have idled for the whole launch.
  auto cut = [](int64_t span, int64_t chunk, bool uneven, int64_t& splits, int64_t& per) {
    splits = 1;
    per = span;
    if (uneven) {
      if (span >= chunk + 64) {
        per = chunk;
        splits = (span + per - 1) / per;
        if (span - (splits - 1) * per < 64) --splits;
      }
      return;
    }
    if (span > chunk + chunk / 4) {
      splits = (span + chunk - 1) / chunk;
      per = round_up((span + splits - 1) / splits, 64);
      splits = (span + per - 1) / per;
    }
  };
  // Longest KV range of one work item.  The grid is (work items x KV heads) CTAs, two resident
  // per SM, handed out longest first by the hardware scheduler; the cost of a candidate limit is
  // the makespan of that list schedule (a CTA costs its tokens plus a fixed prologue/epilogue)
  // plus the split-state traffic of the combine.  Candidates: the throughput heuristic (about
  // four CTAs per resident slot), the longest range divided by small integers, and uneven cuts a
  // little below the longest range.
  int64_t chunk = split_tokens;
  bool uneven = false;
  // The count-only call and the filling call of one plan see the same input: remember the
  // last choice per thread instead of searching twice.
  struct Memo { uint64_t key = 0; int64_t chunk = 0; bool uneven = false; };
  thread_local Memo memo;
  uint64_t key = 1469598103934665603ull;
  auto mix = [&key](uint64_t v) { key = (key ^ v) * 1099511628211ull; };
  for (const Block& b : blocks) { mix((uint64_t)b.n_rows << 32 | (uint32_t)b.lo); mix((uint32_t)b.hi); }
  mix(q_heads); mix(kv_heads); mix(head_dim); mix((uint32_t)window); mix(sm_count);
  if (chunk == 0 && memo.key == key && memo.chunk > 0) {
    chunk = memo.chunk;
    uneven = memo.uneven;
  } else if (chunk == 0) {
    const int64_t slots_resident = (int64_t)sm_count * 2;
    const int64_t want = slots_resident * 4;
    chunk = round_up(std::max<int64_t>(256, (total_span * kv_heads + want - 1) / want), 64);
    int64_t longest = 0;
    for (const Block& b : blocks) longest = std::max<int64_t>(longest, b.hi - b.lo);
    if ((int64_t)blocks.size() * kv_heads < 16 * slots_resident) {
      constexpr double kCtaOverheadTokens = 150.0;    // ~3.5 us of prologue + merge at 23 ns/token
      constexpr double kCombineLaunchTokens = 130.0;  // ~3 us
      constexpr double kLoneSpeedup = 1.5;
      auto estimate = [&](int64_t limit, bool odd) {
        std::vector<int32_t> pieces;
        double combine_bytes = 0.0;
        for (const Block& b : blocks) {
          int64_t splits, per;
          cut(b.hi - b.lo, limit, odd, splits, per);
          for (int64_t i = 0; i < splits; ++i)
            pieces.push_back((int32_t)((i + 1 == splits ? (int64_t)b.hi : b.lo + (i + 1) * per) - (b.lo + i * per)));
          if (splits > 1) combine_bytes += 2.0 * splits * b.n_rows * q_heads * (head_dim + 2) * 4;
        }
        std::sort(pieces.begin(), pieces.end(), std::greater<int32_t>());
        // While CTAs are still queued every slot streams its fair share of the memory bandwidth (rate 1).
        // Once the queue is empty the CTAs that are left speed up as slots fall idle, up to kLoneSpeedup
        // (measured: 36 GB/s for a CTA on an otherwise idle GPU, 23.4 GB/s with all 296 slots busy).
        std::vector<double> heap((size_t)slots_resident, 0.0);       // min-heap of slot finish times at rate 1
        auto later = std::greater<double>();
        double last_start = 0.0;
        for (int32_t len : pieces)
          for (int h = 0; h < kv_heads; ++h) {
            std::pop_heap(heap.begin(), heap.end(), later);
            last_start = heap.back();
            heap.back() += len + kCtaOverheadTokens;
            std::push_heap(heap.begin(), heap.end(), later);
          }
        std::vector<double> left;
        for (double finish : heap)
          if (finish > last_start) left.push_back(finish - last_start);
        std::sort(left.begin(), left.end());
        double makespan = last_start, done = 0.0;
        for (size_t k = 0; k < left.size(); ++k) {
          const double active = (double)(left.size() - k);
          makespan += (left[k] - done) / std::min(kLoneSpeedup, (double)slots_resident / active);
          done = left[k];
        }
        const double token_bytes = 2.0 * head_dim * 2;
        return makespan + combine_bytes / token_bytes / slots_resident + (combine_bytes > 0 ? kCombineLaunchTokens : 0.0);
      };
      double best = estimate(chunk, false);
      for (int k : {1, 2, 3, 4, 6, 8, 12, 16}) {
        const int64_t candidate = round_up((longest + k - 1) / k, 64);
        if (candidate < 256) break;
        // finer cuts than ~12 CTAs per resident slot only add overhead: stop searching there
        int64_t ctas = 0;
        for (const Block& b : blocks) {
          int64_t splits, per;
          cut(b.hi - b.lo, candidate, false, splits, per);
          ctas += splits * kv_heads;
        }
        if (ctas > 12 * slots_resident) break;
        const double cost = estimate(candidate, false);
        if (cost < best * 0.995) {
          best = cost;
          chunk = candidate;
          uneven = false;
        }
      }
      // Uneven cuts: only worth a look while the whole grid is a few waves (that is where idle slots cost most).
      if ((int64_t)blocks.size() * kv_heads <= 4 * slots_resident)
        for (int percent : {97, 94, 91, 88, 85, 80, 75, 70, 65, 60, 55}) {
          const int64_t candidate = round_up(longest * percent / 100, 64);
          if (candidate < 256 || candidate >= longest) continue;
          const double cost = estimate(candidate, true);
          if (cost < best * 0.98) {
            best = cost;
            chunk = candidate;
            uneven = true;
          }
        }
    }
    memo.key = key;
    memo.chunk = chunk;
    memo.uneven = uneven;
  }
  chunk = std::max<int64_t>(chunk, 16);

  struct Item { int32_t w[GK_WORK_WORDS]; };
  std::vector<Item> items;
  std::vector<std::array<int32_t, GK_COMBINE_WORDS>> merges;
  int64_t entries = 0;
  for (const Block& b : blocks) {
    const int64_t span = b.hi - b.lo;
    int64_t splits, per;
    cut(span, chunk, uneven, splits, per);
    if (splits > 0x7fff) return GK_ERR_CAPACITY;     // the split index shares a record word with the count
    int64_t base = -1;
    if (splits > 1) {
      base = entries;
      entries += splits * b.n_rows * q_heads;
      if (entries > INT32_MAX) return GK_ERR_CAPACITY;
      merges.push_back({b.first_row, b.n_rows, (int32_t)base, (int32_t)splits});
    }
    for (int64_t s = 0; s < splits; ++s) {
      Item it{};
      it.w[0] = b.first_row;
      it.w[1] = b.n_rows;
      it.w[2] = b.first_pos;
      it.w[3] = b.table_row;
      it.w[4] = (int32_t)(b.lo + s * per);
      it.w[5] = s + 1 == splits ? b.hi : (int32_t)(b.lo + (s + 1) * per);
      it.w[6] = base < 0 ? -1 : (int32_t)(base + s * b.n_rows * q_heads);
      it.w[7] = (int32_t)(splits | (s << 16));     // low half: splits of the block, high half: which one
      items.push_back(it);
    }
  }
  *n_work_out = (int64_t)items.size();
  *n_combine_out = (int64_t)merges.size();
  *partial_entries_out = entries;
  if (!work_out) return GK_OK;
  if (work_cap < (int64_t)items.size() || combine_cap < (int64_t)merges.size() || (!merges.empty() && !combine_out))
    return GK_ERR_CAPACITY;
  std::stable_sort(items.begin(), items.end(),
                   [](const Item& a, const Item& b) { return a.w[5] - a.w[4] > b.w[5] - b.w[4]; });
  for (size_t i = 0; i < items.size(); ++i) std::copy(items[i].w, items[i].w + GK_WORK_WORDS, work_out + i * GK_WORK_WORDS);
  for (size_t i = 0; i < merges.size(); ++i)
    std::copy(merges[i].begin(), merges[i].end(), combine_out + i * GK_COMBINE_WORDS);
  return GK_OK;
}

extern "C" int gk_prefill_plan_build(const int32_t* seq, int64_t n_seq, int q_heads, int kv_heads, int window,
                                     int min_rows, int32_t* work_out, int64_t work_cap, int64_t* n_work_out,
                                     int32_t* rest_seq_out, int64_t* n_rest_out) {
  if (!seq || n_seq <= 0 || !n_work_out || !n_rest_out || min_rows < 0 || (window != -1 && window <= 0))
    return GK_ERR_INVALID_ARGUMENT;
  if (q_heads <= 0 || kv_heads <= 0 || q_heads % kv_heads != 0 || q_heads / kv_heads > GK_PREFILL_TILE_ROWS)
    return GK_ERR_UNSUPPORTED;
  const int group = q_heads / kv_heads;
  // one record feeds both query tiles of a CTA: up to 2 x (128 / group) consecutive rows
  const int tile_rows = GK_PREFILL_TILES_PER_ITEM * (GK_PREFILL_TILE_ROWS / group);
  if (min_rows == 0) min_rows = std::max(2, (32 + group - 1) / group);
  struct Item { int32_t w[GK_WORK_WORDS]; };
  std::vector<Item> items;
  int64_t n_rest = 0;
  for (int64_t s = 0; s < n_seq; ++s) {
    const int32_t* r = seq + s * 4;
    if (r[1] <= 0 || r[2] < 0 || r[0] < 0 || r[3] < 0) return GK_ERR_INVALID_ARGUMENT;
    if (r[1] < min_rows) {
      if (rest_seq_out) std::copy(r, r + 4, rest_seq_out + n_rest * 4);
      ++n_rest;
      continue;
    }
    for (int32_t done = 0; done < r[1]; done += tile_rows) {
      const int32_t n = std::min<int32_t>(tile_rows, r[1] - done);
      const int64_t first_pos = (int64_t)r[2] + done;
      if (first_pos + n > INT32_MAX) return GK_ERR_UNSUPPORTED;
      Item it{};
      it.w[0] = r[0] + done;
      it.w[1] = n;
      it.w[2] = (int32_t)first_pos;
      it.w[3] = r[3];
      it.w[4] = window > 0 ? (int32_t)std::max<int64_t>(0, first_pos - window + 1) : 0;
      it.w[5] = (int32_t)(first_pos + n);
      it.w[6] = -1;
      it.w[7] = 1;
      items.push_back(it);
    }
  }
  *n_work_out = (int64_t)items.size();
  *n_rest_out = n_rest;
  if (!work_out) return GK_OK;
  if (work_cap < (int64_t)items.size()) return GK_ERR_CAPACITY;
  std::stable_sort(items.begin(), items.end(),
                   [](const Item& a, const Item& b) { return a.w[5] - a.w[4] > b.w[5] - b.w[4]; });
  for (size_t i = 0; i < items.size(); ++i) std::copy(items[i].w, items[i].w + GK_WORK_WORDS, work_out + i * GK_WORK_WORDS);
  return GK_OK;
}
