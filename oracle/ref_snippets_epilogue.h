/* C entry points around the streamed reference functions.  TEST INFRASTRUCTURE ONLY. */
extern "C" {
uint16_t fst_ref_f2bf(float f) { return f2bf(f); }
float fst_ref_bf16f(uint16_t v) { return bf16f(v); }
void fst_ref_rms_cpu(uint16_t* o, const uint16_t* i, const uint16_t* w, int d, int n) {
  rms_cpu(o, i, w, d, n);
}
/* compressed != 0 selects the YaRN branch (a layer whose compress ratio is non-zero). */
void fst_ref_build_rope_lut(uint16_t* lut, int M, int seq_pos, int rope_dim, int compressed,
                            int inverse) {
  FSTEngine e;
  e.config_.rope_dim = rope_dim;
  e.config_.compress_ratios = {compressed ? 4 : 0};
  e.seq_pos_ = seq_pos;
  e.build_rope_lut(lut, M, 0, inverse != 0);
}
}
