/*
 * TEST INFRASTRUCTURE ONLY -- C interface of the CPU oracle.
 * 16-bit values travel as raw uint16_t bit patterns (fp16 or bf16 according to
 * the program's dtype).  dtype: 0 fp16, 1 bf16.  source: 0 current, 1 sollya.
 */
#ifndef FPT_ORACLE_H
#define FPT_ORACLE_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
    FPT_SINCOS_D3_D4_QUARTER_TURN_FP16 = 0,
    FPT_SINCOS_D3_D4_HALF_TURN_FP16,
    FPT_SINCOS_D5_D4_HALF_TURN_FP16,
    FPT_SINCOS_D5_D6_HALF_TURN_FP16,
    FPT_SINCOS_D7_D6_HALF_TURN_FP16,
    FPT_SINCOS_D3_D4_BF16,
    FPT_SINCOS_D3_D4_QUARTER_TURN_BF16,
    FPT_SINCOS_D3_D4_HALF_TURN_BF16,
    FPT_SINCOS_D5_D6_HALF_TURN_BF16,
    FPT_SINCOS_D5_D4_HALF_TURN_FP16_BF16,
    FPT_SINCOS_VARIANT_COUNT
};
enum { FPT_ROPE_HALF_TURN_D5_D6 = 0, FPT_ROPE_QUARTER_TURN_D3_D4 = 1 };

int fpt_oracle_program_count(void);
int fpt_oracle_find_program(const char* name, int dtype, int source);
int fpt_oracle_program_info(int program, char* name_out, int name_cap, int* dtype, int* source,
                            int* shape, int* degree, uint16_t* clamp, uint16_t* coeffs7);
uint16_t fpt_oracle_eval_lane(int program, uint16_t x);

int fpt_oracle_set_threads(int n);
void fpt_oracle_unary(int program, const uint16_t* in, uint16_t* out, int64_t n);
void fpt_oracle_unary_repeat(int program, const uint16_t* in, uint16_t* out, int64_t n, int repeats);
void fpt_oracle_binary_bwd(int program, const uint16_t* grad_out, const uint16_t* x, uint16_t* grad_in, int64_t n);
void fpt_oracle_swiglu(int program, const uint16_t* gate, const uint16_t* up, uint16_t* out, int64_t n);
void fpt_oracle_swiglu_packed(int program, const uint16_t* packed, uint16_t* out, int64_t rows, int64_t hidden);
void fpt_oracle_swiglu_bwd(int fwd_program, int bwd_program, const uint16_t* grad_out, const uint16_t* gate,
                           const uint16_t* up, uint16_t* grad_gate, uint16_t* grad_up, int64_t n);
void fpt_oracle_swiglu_bwd_shared_sigmoid(int sigmoid_program, const uint16_t* grad_out, const uint16_t* gate,
                                          const uint16_t* up, uint16_t* grad_gate, uint16_t* grad_up, int64_t n);

void fpt_oracle_b3_direct_bf16(const uint16_t* scores, uint16_t* prob, uint16_t* grad, int64_t n, int log2_n);
void fpt_oracle_b3_direct_f32(const float* scores, uint16_t* prob, uint16_t* grad, int64_t n, int log2_n);

void fpt_oracle_fma16(const uint16_t* a, const uint16_t* b, const uint16_t* c, uint16_t* out, int64_t n, int dtype);
void fpt_oracle_multiply(const uint16_t* a, const uint16_t* b, uint16_t* out, int64_t n, int dtype);
void fpt_oracle_swish_shared_sigmoid(const uint16_t* x, const uint16_t* s, uint16_t* y, uint16_t* dy, int64_t n, int dtype);
void fpt_oracle_exp2_hinge(const uint16_t* in, uint16_t* out, int64_t n, int set);
int fpt_oracle_sincos_f32(int variant, const float* angles, float* out, int64_t n, int iterations);
void fpt_oracle_exp2_hinge_repeat(const uint16_t* in, uint16_t* out, int64_t n, int set, int repeats);
void fpt_oracle_exp2_full_f32(const float* in, float* out, int64_t n, int variant);

int fpt_oracle_sincos_is_bf16(int variant);
void fpt_oracle_sincos_packed(int variant, const float* angles, uint16_t* cos_out, uint16_t* sin_out, int64_t n);
void fpt_oracle_sincos_packed_compute(int variant, const float* angles, uint16_t* cos_out, uint16_t* sin_out,
                                      int64_t n, int iterations);

void fpt_oracle_rope_table(int kind, const uint32_t* increments, uint16_t* table, int64_t seq, int64_t freq_count);
void fpt_oracle_rope_table_lut(const uint32_t* increments, const uint32_t* lut, uint16_t* table, int64_t seq,
                               int64_t freq_count, int iterations);
void fpt_oracle_rope_apply(const uint16_t* q, const uint16_t* k, const uint32_t* increments, uint16_t* q_out,
                           uint16_t* k_out, int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t D, int io_bf16);

void fpt_oracle_attention_rows(const uint16_t* q, const uint16_t* k, const uint16_t* v, float* out,
                               int64_t B, int64_t S, int64_t Hq, int64_t Hk, int64_t D, int64_t b, int64_t hq,
                               const int64_t* rows, int64_t n_rows, int mode, int causal, float scale,
                               float softcap, int log2_n);

#ifdef __cplusplus
}
#endif
#endif
