// Host entry points for the paged-KV inference kernels (csrc/cuda/decode.cu compiled over cuda_emu.h).
#define NC_EMU
#include "../cuda/decode.cu"

namespace {
using bf = __nv_bfloat16;
template <int D, int G>
void RunDecode(const bf* q, const bf* k_pool, const bf* v_pool, const int* page_table, int max_pages,
               const int* seq_lens, int B, int H, int KV, int page_size, int window_left, float scale, int splits,
               float* part_acc, float* part_ml, bf* out) {
  const float sl2 = scale * 1.4426950408889634f;
  emu::launch(emu::Dim{static_cast<unsigned>(splits), static_cast<unsigned>(KV), static_cast<unsigned>(B)},
              emu::Dim{nc::kDecodeWarps * 32, 1, 1}, 0, [&] {
                nc::paged_decode_kernel<D, G>(q, k_pool, v_pool, page_table, max_pages, seq_lens, H, KV, page_size,
                                              window_left, sl2, splits, part_acc, part_ml, out,
                                              static_cast<long long>(H) * D);
              });
  if (splits > 1)
    emu::launch(emu::Dim{static_cast<unsigned>(H), static_cast<unsigned>(B), 1}, emu::Dim{D, 1, 1}, 0,
                [&] { nc::decode_combine_kernel<D>(part_acc, part_ml, seq_lens, H, splits, out); });
}
}  // namespace

extern "C" {

// Returns 0, or -1 for a shape the kernels do not take. q / out [B, H, D]; pools [pages, page_size, KV, D].
int nc_emu_paged_decode(const void* q, const void* k_pool, const void* v_pool, const int* page_table, int max_pages,
                        const int* seq_lens, int B, int H, int KV, int D, int page_size, int window_left, float scale,
                        int splits, float* part_acc, float* part_ml, void* out) {
  const bf *qq = static_cast<const bf*>(q), *kk = static_cast<const bf*>(k_pool), *vv = static_cast<const bf*>(v_pool);
  bf* oo = static_cast<bf*>(out);
  const int G = H / KV;
#define NC_RUN(DV, GV)                                                                                          \
  RunDecode<DV, GV>(qq, kk, vv, page_table, max_pages, seq_lens, B, H, KV, page_size, window_left, scale, splits, \
                    part_acc, part_ml, oo)
  if (D == 64 && G == 1) NC_RUN(64, 1);
  else if (D == 64 && G == 2) NC_RUN(64, 2);
  else if (D == 128 && G == 1) NC_RUN(128, 1);
  else if (D == 128 && G == 2) NC_RUN(128, 2);
  else if (D == 128 && G == 4) NC_RUN(128, 4);
  else return -1;
#undef NC_RUN
  return 0;
}

void nc_emu_kv_append(void* k_pool, void* v_pool, const int* page_table, int max_pages, const int* positions,
                      const void* k_new, long long k_ld, const void* v_new, long long v_ld, int B, int T, int page_size,
                      int row_elems, int num_pages, int* status) {
  const int total = B * T;
  emu::launch(emu::Dim{static_cast<unsigned>((total + 7) / 8), 1, 1}, emu::Dim{256, 1, 1}, 0, [&] {
    nc::kv_append_kernel(static_cast<bf*>(k_pool), static_cast<bf*>(v_pool), page_table, max_pages, positions,
                         static_cast<const bf*>(k_new), k_ld, static_cast<const bf*>(v_new), v_ld, T, total, page_size,
                         row_elems, num_pages, status);
  });
}

void nc_emu_argmax_rows(const void* logits, long long ld, long long* out, int rows, int vocab) {
  emu::launch(emu::Dim{static_cast<unsigned>(rows), 1, 1}, emu::Dim{256, 1, 1}, 0,
              [&] { nc::argmax_rows_kernel(static_cast<const bf*>(logits), ld, vocab, out); });
}

// Decode prologue (head_dim 128): q and k heads of the fused projection rows normalised, rotated and scaled; k and the
// value row written into their page.
void nc_emu_decode_prep_append(const void* qk, long long ld_qk, const void* v, long long ld_v, const float* cosT,
                               const float* sinT, const int* positions, const int* page_table, int max_pages,
                               int page_size, void* q_out, void* k_pool, void* v_pool, int tokens, int H, int KV,
                               float eps, float scale, int num_pages, int* status) {
  const int groups = (H + KV + 3) / 4;
  const int units = tokens * (groups + 1);
  emu::launch(emu::Dim{static_cast<unsigned>((units + 7) / 8), 1, 1}, emu::Dim{256, 1, 1}, 0, [&] {
    nc::decode_prep_append_kernel(static_cast<const bf*>(qk), ld_qk, static_cast<const bf*>(v), ld_v, cosT, sinT,
                                  positions, page_table, max_pages, page_size, static_cast<bf*>(q_out),
                                  static_cast<bf*>(k_pool), static_cast<bf*>(v_pool), tokens, H, KV, eps, scale,
                                  num_pages, status);
  });
}

void nc_emu_softcap_logits(const void* logits, long long ld, float* out, int rows, int vocab, float cap) {
  const long long pairs = static_cast<long long>(rows) * vocab / 2;
  emu::launch(emu::Dim{static_cast<unsigned>((pairs + 255) / 256), 1, 1}, emu::Dim{256, 1, 1}, 0,
              [&] { nc::softcap_logits_kernel(static_cast<const bf*>(logits), ld, out, rows, vocab, cap); });
}

}  // extern "C"
