// Runs the REFERENCE engine's own Qwen3 graph (CocoRoF/iian: ArchQwen3::build_graph through GraphContext,
// with its paged-attention CPU kernel and a float32 KV cache) on one whole prompt and writes the float32
// logits of every position.  Used only by make_golden.py; linked against the reference's libiian, it is
// not part of the engine.  Modelled on the reference's tests/e2e/test-attn-parity.cpp:24-66 (a hand-built
// UBatch, no engine, no scheduler, no tokenizer).
//
//   reference_logits <model.gguf> <tokens.txt> <out.f32> [flash|softmax|paged]
#include "iian/arch.h"
#include "iian/graph.h"
#include "iian/kv_cache.h"
#include "iian/log.h"
#include "iian/model.h"

#include "ggml-backend.h"
#include "ggml.h"

#include <algorithm>
#include <cstdio>
#include <cstring>
#include <fstream>
#include <stdexcept>
#include <string>
#include <vector>

using namespace iian;

int main(int argc, char ** argv) {
    if (argc < 4) { fprintf(stderr, "usage: %s model.gguf tokens.txt out.f32 [flash|softmax|paged]\n", argv[0]); return 1; }
    const std::string mode = argc > 4 ? argv[4] : "paged";
    Logger::instance().set_level(LogLevel::WARN);
    std::shared_ptr<Model> model = ModelLoader::load(argv[1], DeviceConfig{});
    std::vector<token_t> toks;
    { std::ifstream f(argv[2]); long long t; while (f >> t) toks.push_back((token_t) t); }
    if (toks.empty()) { fprintf(stderr, "no tokens\n"); return 1; }
    const HParams & hp = model->hparams();

    KVCacheConfig kc;
    kc.block_size = 16;
    kc.max_cells = 512;
    kc.type_k = kc.type_v = GGML_TYPE_F32;          // a true 32-bit cache
    kc.enable_prefix_caching = false;
    PagedKVCache kv(*model, kc);
    KVRequestState st;
    if (!kv.allocate_slots(st, (uint32_t) toks.size(), {})) throw std::runtime_error("cache too small");

    UBatch ub;
    ub.n_tokens = (uint32_t) toks.size();
    UBatch::SeqInfo seq;
    for (uint32_t i = 0; i < ub.n_tokens; i++) {
        ub.tokens.push_back(toks[i]);
        ub.pos.push_back((pos_t) i);
        ub.seq_idx.push_back(0);
        ub.slots.push_back(kv.cell_of(st, i));
        ub.out_ids.push_back((int32_t) i);           // logits at every position
        seq.cells.push_back(kv.cell_of(st, i));
        seq.cell_pos.push_back((pos_t) i);
    }
    ub.seqs.push_back(seq);
    ub.n_outputs = ub.n_tokens;
    ub.kv_start = 0;
    ub.n_kv = std::min<uint32_t>(kv.num_cells(), ((uint32_t) (kv.cell_of(st, ub.n_tokens - 1) + 1 + 255) / 256) * 256);

    ggml_backend_t cpu = ggml_backend_dev_init(ggml_backend_dev_by_type(GGML_BACKEND_DEVICE_TYPE_CPU), nullptr);
    ggml_backend_buffer_type_t buft = ggml_backend_get_default_buffer_type(cpu);
    const size_t max_nodes = 16384;
    ggml_backend_sched_t sched = ggml_backend_sched_new(&cpu, &buft, 1, max_nodes, false, true);
    std::vector<uint8_t> meta(ggml_tensor_overhead() * max_nodes + ggml_graph_overhead_custom(max_nodes, false));
    ggml_init_params ip = { meta.size(), meta.data(), true };
    ggml_context * ctx = ggml_init(ip);
    ggml_cgraph * gf = ggml_new_graph_custom(ctx, max_nodes, false);
    GraphContext gc(ctx, gf, *model, ub, kv, /*flash*/ mode != "softmax", /*paged*/ mode == "paged");
    model->arch().build_graph(gc);
    if (!ggml_backend_sched_alloc_graph(sched, gf)) throw std::runtime_error("graph allocation failed");
    gc.set_inputs();
    if (ggml_backend_sched_graph_compute(sched, gf) != GGML_STATUS_SUCCESS) throw std::runtime_error("compute failed");
    std::vector<float> logits((size_t) ub.n_outputs * hp.n_vocab);
    ggml_backend_tensor_get(gc.t_logits, logits.data(), 0, logits.size() * sizeof(float));
    FILE * out = fopen(argv[3], "wb");
    if (!out) throw std::runtime_error("cannot write output");
    fwrite(logits.data(), sizeof(float), logits.size(), out);
    fclose(out);
    printf("%u tokens x %u vocab -> %s (%s)\n", ub.n_tokens, hp.n_vocab, argv[3], mode.c_str());
    ggml_backend_sched_free(sched);
    ggml_free(ctx);
    ggml_backend_free(cpu);
    return 0;
}
