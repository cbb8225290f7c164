// What the kernels of attention_flex*.cu share: the description of one attention call and of the cache it reads.
#pragma once
#include "common.cuh"

#define FLEX_MAX_V 1024   // widest value row of the general kernel

// q is a view [rows, heads, k_dim] with a row stride and a head stride (elements).  Keys: pages
// [page][kv_head][SB_PAGE][k_dim].  Values: pages [page][kv_head][SB_PAGE][v_row] of which the first v_dim columns
// count; for values kept inside the key rows v points at k and v_row is k_dim.  head_scale, slopes and sink are
// 32-bit per query head, null when the option is off; window and chunk are 0 when off.  v_heads: value heads per
// page when they are fewer than key heads (key head c reads value head c / (n_kv_heads / v_heads)); 0 = as many.
// pinned_pages: logical pages that stand before the ring and never turn (the pages of a sequence's kept first tokens).
// keep_first, softcap, talk: read by the kernels of attention_talk.cu only (keys below keep_first stay visible
// outside the window; a scaled score s becomes softcap * tanh(s / softcap); talk [heads, heads] mixes the heads'
// scores); 0 / null = off.
struct SbFlex {
    const void* q;
    long long q_row;
    long long q_head;
    void* k;
    void* v;
    const int* table;
    const float* head_scale;
    const float* slopes;
    const float* sink;
    int table_width;
    int ring_pages;
    int n_heads;
    int n_kv_heads;
    int k_dim;
    int v_dim;
    int v_row;
    int window;
    int chunk;
    float scale;
    int v_heads;
    int pinned_pages;
    int keep_first;
    float softcap;
    const float* talk;
};

// The table column of a logical page: pages before the ring keep their place, later ones turn in the ring.
__device__ __forceinline__ int flex_table_column(const SbFlex& p, int lp) {
    if (!p.ring_pages) return lp;
    return lp < p.pinned_pages ? lp : p.pinned_pages + (lp - p.pinned_pages) % p.ring_pages;
}

// First visible key of a query at position pos.
__device__ __forceinline__ int flex_first_key(const SbFlex& p, int pos) {
    int lo = 0;
    if (p.window > 0) lo = max(lo, pos - p.window + 1);
    if (p.chunk > 0) lo = max(lo, (pos / p.chunk) * p.chunk);
    return lo;
}

// Index of [page][kv_head][pos % SB_PAGE] among a layer's token rows, or -1 when the slot has no page there.
__device__ __forceinline__ long long flex_token(const SbFlex& p, int slot, int pos, int kv_head) {
    const int lp = flex_table_column(p, pos / SB_PAGE);
    if (lp >= p.table_width) return -1;
    const int page = p.table[(long long)slot * p.table_width + lp];
    if (page < 0) return -1;
    return ((long long)page * p.n_kv_heads + kv_head) * SB_PAGE + (pos % SB_PAGE);
}

// The value row that belongs to key row `tok` of key head kv_head (the same row unless value heads are fewer).
__device__ __forceinline__ long long flex_value_token(const SbFlex& p, long long tok, int kv_head) {
    if (p.v_heads <= 0 || p.v_heads == p.n_kv_heads || tok < 0) return tok;
    const long long page = tok / ((long long)p.n_kv_heads * SB_PAGE);
    return (page * p.v_heads + kv_head / (p.n_kv_heads / p.v_heads)) * SB_PAGE + tok % SB_PAGE;
}
// First value row of a page for key head kv_head.
__device__ __forceinline__ long long flex_value_page(const SbFlex& p, int page, int kv_head) {
    if (p.v_heads <= 0 || p.v_heads == p.n_kv_heads) return ((long long)page * p.n_kv_heads + kv_head) * SB_PAGE;
    return ((long long)page * p.v_heads + kv_head / (p.n_kv_heads / p.v_heads)) * SB_PAGE;
}
