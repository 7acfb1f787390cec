/*
 * bunker_tok.h -- C ABI of libbunker_tok.so, the tokenizer boundary of bunker's decode driver.
 *
 * Same entry points and argument meaning as bunker's Rust wrapper around the gigatoken crate
 * (shim/gigatoken_wrapper/src/lib.rs:19-93, bound from TypeScript in prototypes/decode.ts:76-87), implemented in C++
 * over a byte-level BPE read from a Hugging Face tokenizer.json, plus gt_decode, which the reference lacks
 * (prototypes/decode.ts:1071-1078 prints token ids because it cannot turn them back into text).
 */
#ifndef BUNKER_TOK_H
#define BUNKER_TOK_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* lib.rs:19-33 gt_init: path of a tokenizer.json (NUL-terminated); returns a handle, or NULL on any failure. */
void* gt_init(const char* path);
/* lib.rs:35-46 gt_encode: UTF-8 text -> token ids.  Writes at most out_max ids; returns the number written, -1 on a
 * null argument. */
int gt_encode(void* tok, const uint8_t* text, size_t text_len, uint32_t* out_buf, size_t out_max);
/* lib.rs:48-88 gt_encode_mt: the same over chunks cut at spaces and encoded by several threads.  Returns the total
 * number of ids (which may exceed out_max; only ids that fit are written).  Unlike the reference, whose chunks land in
 * completion order, the ids are in text order. */
int gt_encode_mt(void* tok, const uint8_t* text, size_t text_len, uint32_t* out_buf, size_t out_max);
/* No counterpart in the reference: ids -> UTF-8 text.  Writes at most out_max bytes (no terminator); returns the
 * number of bytes the text has (larger than out_max: call again with a bigger buffer), -1 on a null argument. */
int gt_decode(void* tok, const uint32_t* ids, size_t n_ids, uint8_t* out_buf, size_t out_max);
/* Largest token id + 1. */
int gt_vocab_size(void* tok);
/* lib.rs:90-93 gt_free */
void gt_free(void* tok);

#ifdef __cplusplus
}
#endif
#endif /* BUNKER_TOK_H */
