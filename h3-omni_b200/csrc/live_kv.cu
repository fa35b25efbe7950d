// Live mode's KV history as a ring buffer (an addition; the reference keeps it as separately
// allocated tensors that it allocates, copies and frees at every chunk: h3_dit.c:77-80 h3_live_kv,
// live_pair_copy, and the commit at h3_dit.c:4451-4481).
//
// What the history is (h3_dit_live.inc:66-70, h3_dit.c:4457-4481): per layer, the K/V rows of the
// media tokens ([audio | video]) of the last two committed chunks, plus - from the third commit
// on - the video rows of the very first chunk (the "sink"). A chunk's clean K/V is first staged
// ("pending") and becomes history at the commit; the older of the two recent chunks is dropped.
// The media rows of a block then attend  text | sink | older | newer | current media.
//
// Here one allocation per layer holds four slots of chunk_rows rows for K and for V: three rotate
// through the roles pending / newer / older by index, the fourth is the sink. Staging is one device
// copy per tensor (the reference's, too), a commit moves no data except the sink copy of the first
// one, nothing is allocated or freed after h3b_live_kv_new, and attention walks the slots as
// K/V row ranges of the segmented kernel instead of concatenating them first.
#include <new>

#include "attn_kernels.h"
#include "h3_gpu_internal.h"

using h3b::bf16;
using h3b::cuda_good;
using h3b::fail;
using h3b::satisfied;

struct h3b_live_kv {
    h3_gpu *gpu{};
    uint32_t chunk_rows{}, heads{};
    h3_gpu_tensor *key{}, *value{};      // [4][chunk_rows][heads][128]
    struct Slot {
        uint32_t rows, audio, skip;
    } slot[4]{};                          // slot 3: the sink
    int pending{0}, newer{-1}, older{-1};
    bool staged{};
    uint32_t commits{};
};

extern "C" void h3b_live_kv_free(h3b_live_kv *s) {
    if (!s) return;
    h3_gpu_tensor_free(s->key);
    h3_gpu_tensor_free(s->value);
    delete s;
}
extern "C" h3b_live_kv *h3b_live_kv_new(h3_gpu *g, uint32_t chunk_rows, uint32_t heads) {
    if (!g || !chunk_rows || !heads) return nullptr;
    auto *s = new (std::nothrow) h3b_live_kv{};
    if (!s) return nullptr;
    s->gpu = g;
    s->chunk_rows = chunk_rows;
    s->heads = heads;
    const size_t elements = (size_t)4 * chunk_rows * heads * 128;
    s->key = h3b::new_tensor(g, elements, H3_GPU_BF16);
    s->value = h3b::new_tensor(g, elements, H3_GPU_BF16);
    if (!s->key || !s->value) {
        h3b_live_kv_free(s);
        return nullptr;
    }
    return s;
}
extern "C" void h3b_live_kv_reset(h3b_live_kv *s) {
    if (!s) return;
    s->pending = 0;
    s->newer = s->older = -1;
    s->staged = false;
    s->commits = 0;
}
extern "C" uint32_t h3b_live_kv_commits(const h3b_live_kv *s) { return s ? s->commits : 0; }
// Media rows the next attention call will see from the history (sink + the two recent chunks).
extern "C" uint32_t h3b_live_kv_history_rows(const h3b_live_kv *s) {
    if (!s) return 0;
    uint32_t rows = s->commits > 2 ? s->slot[3].rows : 0;
    if (s->older >= 0) rows += s->slot[s->older].rows - s->slot[s->older].skip;
    if (s->newer >= 0) rows += s->slot[s->newer].rows - s->slot[s->newer].skip;
    return rows;
}

static size_t slot_offset(const h3b_live_kv *s, int slot) { return (size_t)slot * s->chunk_rows * s->heads * 128; }

// Stage the clean chunk: rows first_row .. first_row + rows of key / value ([>= first_row + rows]
// [heads][128], the block's K and V after norm + RoPE) are its media rows, the first audio_rows of
// them audio. What live_pair_copy does, into the ring instead of new tensors.
extern "C" int h3b_live_kv_stage(h3b_live_kv *s, const h3_gpu_tensor *key, const h3_gpu_tensor *value, size_t first_row,
                                 uint32_t rows, uint32_t audio_rows) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    if (!rows || rows > s->chunk_rows || audio_rows > rows) {
        fail(g, "live history: a chunk of %u media rows (%u audio) does not fit slots of %u rows", rows, audio_rows,
             s->chunk_rows);
        return 0;
    }
    const size_t width = (size_t)s->heads * 128, n = (size_t)rows * width;
    if (!satisfied(g, {bf16(key, (first_row + rows) * width, "live key"), bf16(value, (first_row + rows) * width, "live value")}))
        return 0;
    const size_t at = slot_offset(s, s->pending);
    if (!h3_gpu_copy_bf16(g, s->key, at, key, first_row * width, n) ||
        !h3_gpu_copy_bf16(g, s->value, at, value, first_row * width, n))
        return 0;
    s->slot[s->pending] = {rows, audio_rows, 0};
    s->staged = true;
    return 1;
}

// The staged chunk becomes the newest history chunk, the older of the two recent chunks is
// dropped (its slot is the next staging slot). The first commit also retains the chunk's video rows
// as the sink: the only data a commit moves.
extern "C" int h3b_live_kv_commit(h3b_live_kv *s) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    if (!s->staged) {
        fail(g, "incomplete live clean commit");
        return 0;
    }
    if (!s->commits) {
        const h3b_live_kv::Slot &p = s->slot[s->pending];
        const size_t width = (size_t)s->heads * 128, n = (size_t)(p.rows - p.audio) * width;
        const size_t from = slot_offset(s, s->pending) + (size_t)p.audio * width, to = slot_offset(s, 3);
        if (n && (!h3_gpu_copy_bf16(g, s->key, to, s->key, from, n) || !h3_gpu_copy_bf16(g, s->value, to, s->value, from, n)))
            return 0;
        s->slot[3] = {p.rows - p.audio, 0, 0};
    }
    const int freed = s->older >= 0 ? s->older : (s->newer >= 0 ? 3 - s->pending - s->newer : (s->pending + 1) % 3);
    s->older = s->newer;
    s->newer = s->pending;
    s->pending = freed;
    s->staged = false;
    s->commits++;
    return 1;
}
// From now on the two recent chunks are attended without their audio rows (h3_dit.c:4483-4486).
extern "C" int h3b_live_kv_clear_audio(h3b_live_kv *s) {
    if (!s) return 0;
    for (int slot : {s->older, s->newer})
        if (slot >= 0) s->slot[slot].skip = s->slot[slot].audio;
    return 1;
}

// The media rows of a block against  text | sink | older | newer | current media  (the second call
// of h3_dit_live.inc:95-99), without the concatenation copies of :81-94. key / value hold the
// block's own rows [sequence][heads][128] with the text rows first; query rows q_row .. + query_rows
// are written to out rows out_row .. .
extern "C" int h3b_live_kv_attention_bf16(h3b_live_kv *s, h3_gpu_tensor *out, size_t out_row, const h3_gpu_tensor *q,
                                          size_t q_row, uint32_t query_rows, const h3_gpu_tensor *key,
                                          const h3_gpu_tensor *value, uint32_t text_rows, uint32_t sequence) {
    if (!s) return 0;
    h3_gpu *g = s->gpu;
    if (text_rows > sequence || !sequence) {
        fail(g, "live history attention: %u text rows of %u", text_rows, sequence);
        return 0;
    }
    const h3_gpu_tensor *keys[6], *values[6];
    size_t first[6];
    uint32_t rows[6], count = 0;
    auto add = [&](const h3_gpu_tensor *k, const h3_gpu_tensor *v, size_t start, uint32_t n) {
        if (!n) return;
        keys[count] = k;
        values[count] = v;
        first[count] = start;
        rows[count++] = n;
    };
    add(key, value, 0, text_rows);
    if (s->commits > 2) add(s->key, s->value, (size_t)3 * s->chunk_rows, s->slot[3].rows);
    for (int slot : {s->older, s->newer})
        if (slot >= 0)
            add(s->key, s->value, (size_t)slot * s->chunk_rows + s->slot[slot].skip, s->slot[slot].rows - s->slot[slot].skip);
    add(key, value, text_rows, sequence - text_rows);
    return h3b_cross_attention_segments_bf16(g, out, out_row, q, q_row, query_rows, s->heads, count, keys, values, first, rows);
}
