// b200_serve: command line of the model-family layer (include/b200_serve.h).
//
//   b200_serve trace    --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--slots S]
//       replays steps read from standard input, one JSON object per line:
//         {"step": 0, "entries": [{"id": "a", "tokens": [5, 17, 3], "want": [0, 2]}], "end": ["a"]}
//       All entries of a line run as one batch through the engine's step function. When places are wanted the logits
//       go to DIR/<step>.f32 (little-endian fp32 [wanted, vocab], in the order of the entries and of "want"); after
//       every step "done <step>" is printed. Requests named in "end" give their slot and pages back.
//   b200_serve generate --model DIR [--dtype ...] --prompt 1,2,3 [--prompt ...] [--max-new N] [--eos ID] [--chunk C]
//                       [--slots S] [--max-tokens N]
//       greedy generation of all prompts through the continuous-batching scheduler; prints one line of ids per prompt.
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <iostream>
#include <string>
#include <vector>

#include "b200_serve.h"
#include "json_min.h"

using b200::Json;

static int usage() {
    fprintf(stderr, "usage: b200_serve trace --model DIR --dtype bfloat16|float32 --out DIR --max-tokens N [--slots S]\n"
                    "       b200_serve generate --model DIR --prompt IDS [--prompt IDS ...] [--max-new N] [--eos ID] [--chunk C]\n"
                    "                           [--dtype bfloat16|float32] [--slots S] [--max-tokens N]\n");
    return 2;
}

static int run_trace(b200_model* m, const std::string& out_dir) {
    b200_session* ses = b200_session_create(m);
    const int V = b200_model_vocab(m);
    std::string line, err;
    std::vector<int> slots, counts, tokens, n_want, want;
    std::vector<float> logits;
    while (std::getline(std::cin, line)) {
        if (line.find_first_not_of(" \t\r\n") == std::string::npos) continue;
        Json j;
        if (!b200::JsonParser::parse(line.data(), line.size(), j, err)) { fprintf(stderr, "trace: %s\n", err.c_str()); return 1; }
        const long long step = j.integer("step", -1);
        const Json* en = j.get("entries");
        slots.clear(); counts.clear(); tokens.clear(); n_want.clear(); want.clear();
        if (en && en->kind == Json::Arr)
            for (const Json& e : en->arr) {
                const std::string id = e.text("id");
                const Json* tk = e.get("tokens");
                const Json* wt = e.get("want");
                if (!tk || tk->kind != Json::Arr || tk->arr.empty()) continue;   // nothing to run for this request now
                const int slot = b200_session_slot(ses, id.c_str());
                if (slot < 0) { fprintf(stderr, "trace: %s\n", b200_serve_last_error()); return 1; }
                slots.push_back(slot);
                counts.push_back((int)tk->arr.size());
                for (const Json& t : tk->arr) tokens.push_back((int)t.num);
                int nw = 0;
                if (wt && wt->kind == Json::Arr)
                    for (const Json& w : wt->arr) { want.push_back((int)w.num); ++nw; }
                n_want.push_back(nw);
            }
        const size_t total_want = want.size();
        logits.resize(total_want * V);
        if (!slots.empty()) {
            const int rc = b200_model_step(m, (int)slots.size(), slots.data(), counts.data(), tokens.data(), n_want.data(), want.data(),
                                           total_want ? logits.data() : nullptr, nullptr);
            if (rc != 0) { fprintf(stderr, "trace: step %lld failed (%d): %s\n", step, rc, b200_serve_last_error()); return 1; }
        }
        if (total_want) {
            const std::string path = out_dir + "/" + std::to_string(step) + ".f32";
            FILE* f = fopen(path.c_str(), "wb");
            if (!f || fwrite(logits.data(), sizeof(float), logits.size(), f) != logits.size()) { fprintf(stderr, "trace: cannot write %s\n", path.c_str()); return 1; }
            fclose(f);
        }
        const Json* end = j.get("end");
        if (end && end->kind == Json::Arr)
            for (const Json& e : end->arr)
                if (e.kind == Json::Str) b200_session_end(ses, e.str.c_str());
        printf("done %lld\n", step);
        fflush(stdout);
    }
    b200_session_destroy(ses);
    return 0;
}

int main(int argc, char** argv) {
    if (argc < 2) return usage();
    const std::string cmd = argv[1];
    std::string model, out, dtype = "bfloat16";
    std::vector<std::vector<int>> prompts;
    int max_tokens = 0, slots = 4, max_new = 16, eos = -1, chunk = 0;
    for (int i = 2; i < argc; ++i) {
        const std::string a = argv[i];
        auto val = [&]() -> const char* { return i + 1 < argc ? argv[++i] : ""; };
        if (a == "--model") model = val();
        else if (a == "--out") out = val();
        else if (a == "--dtype") dtype = val();
        else if (a == "--max-tokens") max_tokens = atoi(val());
        else if (a == "--slots") slots = atoi(val());
        else if (a == "--max-new") max_new = atoi(val());
        else if (a == "--eos") eos = atoi(val());
        else if (a == "--chunk") chunk = atoi(val());
        else if (a == "--prompt") {
            std::vector<int> p;
            const char* s = val();
            while (*s) {
                char* e;
                const long v = strtol(s, &e, 10);
                if (e == s) break;
                p.push_back((int)v);
                s = *e ? e + 1 : e;
            }
            prompts.push_back(p);
        } else
            return usage();
    }
    if (model.empty() || (dtype != "bfloat16" && dtype != "float32")) return usage();
    b200_model_options opt{};
    opt.dtype = dtype == "float32" ? B200_F32 : B200_BF16;
    opt.max_slots = slots;
    if (cmd == "trace") {
        if (out.empty() || max_tokens < 1) return usage();
        opt.max_tokens = max_tokens;
        b200_model* m = b200_model_open(model.c_str(), &opt);
        if (!m) { fprintf(stderr, "b200_serve: %s\n", b200_serve_last_error()); return 1; }
        const int rc = run_trace(m, out);
        b200_model_close(m);
        return rc;
    }
    if (cmd == "generate") {
        if (prompts.empty()) return usage();
        std::vector<int> ids, lens;
        size_t need = 0;
        for (auto& p : prompts) {
            if (p.empty()) return usage();
            ids.insert(ids.end(), p.begin(), p.end());
            lens.push_back((int)p.size());
            need += (p.size() + max_new + 63) / 64 * 64;
        }
        opt.max_tokens = max_tokens > 0 ? max_tokens : (int)need;
        b200_model* m = b200_model_open(model.c_str(), &opt);
        if (!m) { fprintf(stderr, "b200_serve: %s\n", b200_serve_last_error()); return 1; }
        std::vector<int> outv(prompts.size() * (size_t)max_new), made(prompts.size());
        const int rc = b200_model_generate(m, (int)prompts.size(), ids.data(), lens.data(), max_new, eos, chunk, outv.data(), made.data());
        if (rc < 0) { fprintf(stderr, "b200_serve: generate failed (%d): %s\n", rc, b200_serve_last_error()); b200_model_close(m); return 1; }
        for (size_t r = 0; r < prompts.size(); ++r) {
            for (int k = 0; k < made[r]; ++k) printf("%s%d", k ? " " : "", outv[r * max_new + k]);
            printf("\n");
        }
        fprintf(stderr, "%s: %d engine steps\n", b200_model_family(m), rc);
        b200_model_close(m);
        return 0;
    }
    return usage();
}
