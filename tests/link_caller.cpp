// A caller of the library written against the REFERENCE's public header (compiled with -I<reference>/include,
// never against this repository's own header) and linked with -lkutacc: it shows that a program built for
// the reference links and runs against this library unchanged - struct layouts, the mangled
// kutacc::TensorWrapper constructor and destructor, default visibility of the C symbols.
//
//   link_caller null                       the robustness path: one null handle, nothing is dereferenced
//   link_caller run <in.bin> <out.bin>     one small gated-attention call on host buffers read from <in.bin>
//
// <in.bin>: int64 header {B, S, H, D, has_nb}, then bf16 x [B*S*C], wq, wk, wv, wg, wo [C*C each], fp32 bg, bo [C],
// bf16 bias [B*S], bf16 nb [H*S*S] (when has_nb). <out.bin>: bf16 out [B*S*C].
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "kutacc.h"

using kutacc::kBF16;
using kutacc::TensorWrapper;

static std::vector<char> slurp(const char *path)
{
    std::vector<char> buf;
    FILE *f = std::fopen(path, "rb");
    if (!f) return buf;
    std::fseek(f, 0, SEEK_END);
    const long n = std::ftell(f);
    std::fseek(f, 0, SEEK_SET);
    buf.resize((size_t)n);
    if (std::fread(buf.data(), 1, (size_t)n, f) != (size_t)n) buf.clear();
    std::fclose(f);
    return buf;
}

int main(int argc, char **argv)
{
    kutacc_version_t v;
    if (kutacc_get_version(&v) != KUTACC_OK) return 2;
    std::printf("linked against %s %s\n", v.component_name, v.component_version);
    if (argc >= 2 && std::strcmp(argv[1], "null") == 0) {
        float a = 0.8f;                         // as the reference's own robustness tests do: a stack float as a handle
        void *h = &a;
        kutacc_af2_attention_inputs_t in = {2, 2, h, h, h, h, h};
        kutacc_af2_attention_weights_t w = {2, 1, 2, h, h, h, h, h, h, h};
        kutacc_af2_gating_attention(nullptr, &in, h, h, &w, h, 1);
        std::printf("null handle reported\n");
        return 0;
    }
    if (argc < 4 || std::strcmp(argv[1], "run") != 0) return 3;
    std::vector<char> buf = slurp(argv[2]);
    if (buf.size() < 5 * sizeof(int64_t)) return 4;
    int64_t hdr[5];
    std::memcpy(hdr, buf.data(), sizeof(hdr));
    const int64_t B = hdr[0], S = hdr[1], H = hdr[2], D = hdr[3], has_nb = hdr[4], C = H * D;
    char *p = buf.data() + sizeof(hdr);
    auto take = [&](size_t bytes) { char *q = p; p += bytes; return (void *)q; };
    void *x = take((size_t)B * S * C * 2);
    void *wq = take((size_t)C * C * 2), *wk = take((size_t)C * C * 2), *wv = take((size_t)C * C * 2),
         *wg = take((size_t)C * C * 2), *wo = take((size_t)C * C * 2);
    void *bg = take((size_t)C * 4), *bo = take((size_t)C * 4);
    void *bias = take((size_t)B * S * 2);
    void *nb = has_nb ? take((size_t)H * S * S * 2) : nullptr;
    if ((size_t)(p - buf.data()) > buf.size()) return 5;
    std::vector<uint16_t> out((size_t)B * S * C), scratch((size_t)B * S * C);
    {
        TensorWrapper t_x(x, {B * S, C}, {C, 1}, 2, kBF16), t_out(out.data(), {B, S, C}, {S * C, C, 1}, 3, kBF16);
        TensorWrapper t_wq(wq, {C, C}, {C, 1}, 2, kBF16), t_wk(wk, {C, C}, {C, 1}, 2, kBF16), t_wv(wv, {C, C}, {C, 1}, 2, kBF16),
            t_wg(wg, {C, C}, {C, 1}, 2, kBF16), t_wo(wo, {C, C}, {C, 1}, 2, kBF16);
        TensorWrapper t_bg(bg, {C}, {1}, 1, kBF16), t_bo(bo, {C}, {1}, 1, kBF16);   // the reference has no fp32 tag
        TensorWrapper t_bias(bias, {B, S}, {S, 1}, 2, kBF16);
        TensorWrapper t_nb = has_nb ? TensorWrapper(nb, {H, S, S}, {S * S, S, 1}, 3, kBF16)
                                    : TensorWrapper(nullptr, {0}, {1}, 1, kBF16);
        TensorWrapper t_s(scratch.data(), {B, S, H, D}, {S * C, C, D, 1}, 4, kBF16);
        kutacc_af2_attention_inputs_t in = {B, S, t_s.get_tensor(), t_s.get_tensor(), t_s.get_tensor(), t_s.get_tensor(),
                                            t_s.get_tensor()};
        kutacc_af2_attention_weights_t w = {C, H, D, t_wq.get_tensor(), t_wk.get_tensor(), t_wv.get_tensor(),
                                            t_wg.get_tensor(), t_bg.get_tensor(), t_wo.get_tensor(), t_bo.get_tensor()};
        kutacc_af2_gating_attention(t_x.get_tensor(), &in, t_bias.get_tensor(), t_nb.get_tensor(), &w, t_out.get_tensor(), 128);
    }
    FILE *f = std::fopen(argv[3], "wb");
    if (!f) return 6;
    std::fwrite(out.data(), 2, out.size(), f);
    std::fclose(f);
    std::printf("wrote %zu values\n", out.size());
    return 0;
}
