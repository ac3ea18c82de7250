/* Minimal declarations of the public PCRE2 8-bit API -- TEST INFRASTRUCTURE ONLY.
 * The image carries the PCRE2 runtime library (libpcre2-8.so.0) but not its development header.
 * The reference's tokenizer (src/tokenizer.cpp:10-65) uses exactly the calls declared here, so this
 * stand-in lets the oracle build compile that file unmodified and link it against the system's
 * runtime library.  Names, argument types and the three option values follow PCRE2's documented
 * C interface (pcre2api(3)); nothing here is PCRE2 code. */
#ifndef SLLM_ORACLE_PCRE2_DECL_H
#define SLLM_ORACLE_PCRE2_DECL_H
#include <stddef.h>
#include <stdint.h>
#ifdef __cplusplus
extern "C" {
#endif
typedef const uint8_t* PCRE2_SPTR;
typedef size_t PCRE2_SIZE;
typedef struct pcre2_real_code_8 pcre2_code;
typedef struct pcre2_real_match_data_8 pcre2_match_data;
typedef struct pcre2_real_general_context_8 pcre2_general_context;
typedef struct pcre2_real_compile_context_8 pcre2_compile_context;
typedef struct pcre2_real_match_context_8 pcre2_match_context;
#define PCRE2_ZERO_TERMINATED (~(PCRE2_SIZE)0)
#define PCRE2_UTF 0x00080000u
#define PCRE2_UCP 0x00020000u
#define PCRE2_JIT_COMPLETE 0x00000001u
pcre2_code* pcre2_compile_8(PCRE2_SPTR, PCRE2_SIZE, uint32_t, int*, PCRE2_SIZE*, pcre2_compile_context*);
int pcre2_jit_compile_8(pcre2_code*, uint32_t);
pcre2_match_data* pcre2_match_data_create_from_pattern_8(const pcre2_code*, pcre2_general_context*);
int pcre2_match_8(const pcre2_code*, PCRE2_SPTR, PCRE2_SIZE, PCRE2_SIZE, uint32_t, pcre2_match_data*, pcre2_match_context*);
int pcre2_jit_match_8(const pcre2_code*, PCRE2_SPTR, PCRE2_SIZE, PCRE2_SIZE, uint32_t, pcre2_match_data*, pcre2_match_context*);
PCRE2_SIZE* pcre2_get_ovector_pointer_8(pcre2_match_data*);
void pcre2_match_data_free_8(pcre2_match_data*);
void pcre2_code_free_8(pcre2_code*);
#define pcre2_compile pcre2_compile_8
#define pcre2_jit_compile pcre2_jit_compile_8
#define pcre2_match_data_create_from_pattern pcre2_match_data_create_from_pattern_8
#define pcre2_match pcre2_match_8
#define pcre2_jit_match pcre2_jit_match_8
#define pcre2_get_ovector_pointer pcre2_get_ovector_pointer_8
#define pcre2_match_data_free pcre2_match_data_free_8
#define pcre2_code_free pcre2_code_free_8
#ifdef __cplusplus
}
#endif
#endif
