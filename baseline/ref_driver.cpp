// Drives the unmodified vt-transformer v1 engine (libtensortype, its CUDA kernels, cuBLASLt, cuDNN) on its own
// graph v1/models/qwen2-7b/inference_fp16.dag, the way v1/models/qwen2-7b/chat.cpp:87-111 and :186-224 do: the
// graph text is built and run with "cuda" on the stack, "gpu_init" loads the weights, and every step writes the
// whole token list and its mask into the in-process pipe, pushes (batch, length) and runs "gpu_main", which
// answers with the sampled ids through the pipe.  There is no tokenizer here (chat.cpp needs it for text only)
// and the weights are raw fp16 files of random numbers with the names and sizes the graph loads (:87-142).
//
// Graph files are concatenated as chat.cpp's main() concatenates its arguments, so a second file may set
// MAX_BATCH after the first has set it to 1.
//
//   ref_driver --dag FILE [--dag FILE2] --batch B --prompt-len P --steps K --warmup W --prefill T --prefill-runs R
//
// It prints one line: {"decode_ms_per_step": .., "decode_tok_s": .., "prefill_ms": .., "prefill_ms_all": [..]}.
// Times are wall-clock around whole steps with the device idle on both sides: a step of this engine is host
// work (matching the token list against its cache, copies of the cache into contiguous buffers) and kernels.
#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <fcntl.h>
#include <fstream>
#include <iostream>
#include <random>
#include <string>
#include <unistd.h>
#include <vector>

#include <tensortype_inc.hpp>

#include "memory.hpp"

static std::string file_text(const char* name) {
    std::ifstream t(name);
    if (!t.is_open()) {
        std::cerr << "ref_driver: cannot open " << name << std::endl;
        exit(2);
    }
    return std::string((std::istreambuf_iterator<char>(t)), std::istreambuf_iterator<char>());
}

struct Driver {
    vt::ComputingContext* ctx;
    vt::Enviroment* env;
    vt::DaG* main_code;
    int vocab;
    std::mt19937 rng{12345};

    std::vector<int> random_tokens(size_t n) {
        std::vector<int> v(n);
        for (auto& x : v) x = (int)(rng() % (unsigned)vocab);
        return v;
    }

    // One run of gpu_main over `batch` sequences of `len` tokens each (row-major ids); returns the sampled ids.
    std::vector<int> step(int batch, int len, const std::vector<int>& ids) {
        std::vector<int> mask((size_t)batch * len, 1);
        for (int b = 0; b < batch; b++) mask[(size_t)b * len + len - 1] = 2;
        if (ctx->pipe_write(0, ids.data(), ids.size() * sizeof(int)) != (int)(ids.size() * sizeof(int)) ||
            ctx->pipe_write(0, mask.data(), mask.size() * sizeof(int)) != (int)(mask.size() * sizeof(int))) {
            std::cerr << "ref_driver: short write into the pipe" << std::endl;
            exit(3);
        }
        env->stack().push_number(batch);
        env->stack().push_number(len);
        env->run(main_code);
        std::vector<int> next(batch, -1);
        ctx->pipe_read(next.data(), batch * sizeof(int));
        return next;
    }
};

static double now_ms() {
    return std::chrono::duration<double, std::milli>(std::chrono::steady_clock::now().time_since_epoch()).count();
}

int main(int argc, const char* argv[]) {
    std::vector<std::string> dags;
    int batch = 1, prompt_len = 1024, steps = 20, warmup = 3, prefill = 2048, prefill_runs = 3;
    for (int i = 1; i + 1 < argc; i += 2) {
        std::string k = argv[i];
        if (k == "--dag") dags.push_back(argv[i + 1]);
        else if (k == "--batch") batch = atoi(argv[i + 1]);
        else if (k == "--prompt-len") prompt_len = atoi(argv[i + 1]);
        else if (k == "--steps") steps = atoi(argv[i + 1]);
        else if (k == "--warmup") warmup = atoi(argv[i + 1]);
        else if (k == "--prefill") prefill = atoi(argv[i + 1]);
        else if (k == "--prefill-runs") prefill_runs = atoi(argv[i + 1]);
        else { std::cerr << "ref_driver: unknown option " << k << std::endl; return 2; }
    }
    if (dags.empty()) { std::cerr << "ref_driver: --dag FILE is needed" << std::endl; return 2; }

    vt::ComputingContext* ctx = new vt::ComputingContext();
    ctx->boot_host(0);
    ctx->boot_cuda(0);
    // a step's token list and mask lie in the pipe together before the graph reads them: make room for them
    for (int fd : ctx->pipe_fds) {
        if (fd >= 0) fcntl(fd, F_SETPIPE_SZ, 1 << 20);
    }
    vt::Enviroment* env = new vt::Enviroment(ctx);
    env->insert_native_word("app.mem", MemoryCounting::creator);
    env->insert_native_word("app.align", MemoryAlign::creator);
    {
        std::string all_code;
        for (auto& d : dags) all_code += file_text(d.c_str()) + "\n";
        vt::DaG* init_bin = env->build(all_code);
        env->stack().push_string("cuda");
        env->run(init_bin);
        delete init_bin;
    }
    env->execute("gpu_init");

    Driver d{ctx, env, env->build("gpu_main"), 152064};
    size_t need = (size_t)batch * (prompt_len + warmup + steps + 1) * sizeof(int) * 2;
    if (need > (1u << 20)) { std::cerr << "ref_driver: a step's ids and mask exceed the pipe" << std::endl; return 2; }

    // prefill: one sequence of `prefill` fresh tokens, whole, logits of the last token
    std::vector<double> prefill_ms;
    for (int r = 0; r < prefill_runs + 1 && prefill > 0; r++) {
        auto ids = d.random_tokens(prefill);
        cudaDeviceSynchronize();
        double t0 = now_ms();
        d.step(1, prefill, ids);
        cudaDeviceSynchronize();
        double t1 = now_ms();
        if (r > 0) prefill_ms.push_back(t1 - t0);          // the first run is the warm-up
    }

    // decode: `batch` sequences of `prompt_len` tokens, then one token each a step; every step sends the whole lists
    int len = prompt_len;
    std::vector<std::vector<int>> seqs(batch);
    for (auto& s : seqs) s = d.random_tokens(prompt_len);
    auto flat = [&]() {
        std::vector<int> ids;
        ids.reserve((size_t)batch * len);
        for (auto& s : seqs) ids.insert(ids.end(), s.begin(), s.end());
        return ids;
    };
    auto advance = [&](const std::vector<int>& next) {
        for (int b = 0; b < batch; b++) seqs[b].push_back(next[b] >= 0 && next[b] < d.vocab ? next[b] : 0);
        len++;
    };
    advance(d.step(batch, len, flat()));                    // the prompts
    for (int i = 0; i < warmup; i++) advance(d.step(batch, len, flat()));
    cudaDeviceSynchronize();
    double t0 = now_ms();
    for (int i = 0; i < steps; i++) advance(d.step(batch, len, flat()));
    cudaDeviceSynchronize();
    double t1 = now_ms();

    std::sort(prefill_ms.begin(), prefill_ms.end());
    double pm = prefill_ms.empty() ? 0.0 : prefill_ms[prefill_ms.size() / 2];
    printf("{\"decode_ms_per_step\": %.4f, \"decode_tok_s\": %.2f, \"batch\": %d, \"steps\": %d, \"context_end\": %d, "
           "\"prefill_ms\": %.3f, \"prefill_tokens\": %d, \"prefill_ms_all\": [",
           (t1 - t0) / steps, batch * steps / ((t1 - t0) / 1e3), batch, steps, len, pm, prefill);
    for (size_t i = 0; i < prefill_ms.size(); i++) printf("%s%.3f", i ? ", " : "", prefill_ms[i]);
    printf("]}\n");
    fflush(stdout);
    _exit(0);      // the engine's tensors are released by the process's end, as chat.cpp leaves them
}
