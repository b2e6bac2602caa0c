/* TEST INFRASTRUCTURE ONLY (force-included when oracle/build_ref.py compiles the reference's
 * compiler/runtime/tokenizer.cpp). Without MLC_ENABLE_LLAMA_TOKENIZER that file takes its own BPE / unigram /
 * greedy code paths, but four llama.cpp calls in its constructor (tokenizer.cpp:42-54, reached only when
 * use_llama_cpp_ is true, which tryInitLlamaCpp leaves false) are not behind the macro and need declarations to
 * compile. llama.cpp itself is not vendored in the reference tree; these are declarations only - the definitions
 * are the generated return-zero stubs, never called. */
#pragma once
#ifdef __cplusplus
extern "C" {
#endif
struct llama_vocab;
int llama_vocab_n_tokens(const struct llama_vocab* vocab);
const char* llama_vocab_get_text(const struct llama_vocab* vocab, int token);
int llama_vocab_bos(const struct llama_vocab* vocab);
int llama_vocab_eos(const struct llama_vocab* vocab);
#ifdef __cplusplus
}
#endif
