"""Generates full_models.npz: greedy ids and logits of the benchmark configurations AT FULL SIZE from
the REFERENCE's own CPU code (oracle/_ref/libref_cpu.so = the unmodified reference sources), plus the
INT8-KV variants from the restated oracle (oracle.c; the reference has no CPU INT8 cache).

  python tests/golden/make_golden_full.py [c1] [c2] [c3]        (hours of CPU time in total)

Protocol per configuration (weights = the package's seeded synthetic GGUF of the named shape):
  c1  TinyLlama-1.1B shape, every linear Q8_0, FP32 KV: 128-token prompt, 32 greedy steps
  c2  TinyLlama-1.1B shape, Q4_K_M-style, 512-token prompt, 32 greedy steps, FP32 KV (reference)
      and INT8 KV (restated oracle)
  c3  Llama-2-7B shape, Q4_K_M-style, SHORTENED: 32-token prompt, 8 greedy steps, FP32 KV (reference)
      and INT8 KV (restated oracle); a 7B token costs the reference about 20 s of CPU time
Prompts: token ids uniform in [0, vocab) from PCG64(4321) (sequence 0 of the benchmark). The prompt
goes through the reference's batch path (forward_cpu_batch, as its session does for >= 32 tokens),
the steps through forward(). Stored per case: prompt, logits after the prompt, the greedy ids, the
logits of the first / middle / last step, and the top-2 gap of every step (so a test can tell a
genuine mismatch from a near-tie).
"""
import os
import sys
import time

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))
import oracle_lib as ol  # noqa: E402

pkg = ol.pkg

CASES = {
    # name: (shape, scheme, prompt_len, steps)
    "c1": ("tinyllama-1.1b", 0, 128, 32),
    "c2": ("tinyllama-1.1b", 1, 512, 32),
    "c3": ("llama2-7b", 1, 32, 8),
}


def model_file(shape, scheme):
    base = "/dev/shm" if os.path.isdir("/dev/shm") else "/tmp"
    path = os.path.join(base, f"b200_synth_{shape}_s{scheme}.gguf")
    if not os.path.exists(path):
        pkg.synth.write_gguf(path + ".tmp", shape, scheme=scheme)
        os.replace(path + ".tmp", path)
    return path


def run(model, prompt, steps, tag, fx):
    t0 = time.time()
    out = model.prefill(prompt)
    fx[f"{tag}_prefill_logits"] = out.copy()
    print(tag, "prefill", round(time.time() - t0, 1), "s", flush=True)
    keep = sorted({0, steps // 2 - 1 if steps > 2 else 0, steps - 1})
    tok, ids, gaps, lg = int(out.argmax()), [], [], []
    top = np.sort(out)[-2:]
    first_gap = float(top[1] - top[0])
    for i in range(steps):
        ids.append(tok)
        out = model.decode(tok, len(prompt) + i)
        top = np.sort(out)[-2:]
        gaps.append(float(top[1] - top[0]))
        if i in keep:
            lg.append(out.copy())
        tok = int(out.argmax())
        print(tag, "step", i, tok, round(time.time() - t0, 1), "s", flush=True)
    fx[f"{tag}_ids"] = np.array(ids + [tok], np.int32)          # ids[0] = argmax after the prompt, then one per step
    fx[f"{tag}_gaps"] = np.array([first_gap] + gaps, np.float32)
    fx[f"{tag}_step_index"] = np.array(keep, np.int32)
    fx[f"{tag}_step_logits"] = np.stack(lg)


def main():
    which = [a for a in sys.argv[1:] if a in CASES] or list(CASES)
    out_path = os.path.join(HERE, "full_models.npz")
    fx = dict(np.load(out_path)) if os.path.exists(out_path) else {}
    for name in which:
        shape, scheme, n_prompt, steps = CASES[name]
        path = model_file(shape, scheme)
        vocab = pkg.synth.SHAPES[shape]["vocab"]
        prompt = np.random.Generator(np.random.PCG64(4321)).integers(0, vocab, n_prompt).astype(np.int32)
        fx[f"{name}_prompt"] = prompt
        r = ol.RefModel(path)
        run(r, prompt, steps, f"{name}_f32", fx)
        del r
        np.savez_compressed(out_path, **fx)
        if name != "c1":
            o = ol.OracleModel.from_gguf(path, kv_int8=True)
            run(o, prompt, steps, f"{name}_i8", fx)
            del o
            np.savez_compressed(out_path, **fx)
    print("wrote", out_path, sorted(fx))


if __name__ == "__main__":
    main()
