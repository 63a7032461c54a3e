#!/usr/bin/env python3
"""Makes the files under tests/golden/reference_fixture*/ with the reference's own code, on the CPU.

What it does, from the root of this repository:
  1. builds ktfth/smolmoe-c99's CLI with the machine's C compiler (its Makefile, build folder
     under /tmp: the reference tree is not written to);
  2. writes tiny random `smolmoe_qwen2` checkpoints with the reference's own
     tools/checkpoint.py (`fixture`): reference_fixture -- 2 layers, dim 64, 4 heads, 2 kv
     heads (head size 16), hidden 128, vocabulary 258, rope base 1e4, eps 1e-6, seed 11;
     reference_fixture_b -- 3 layers, dim 96, 3 heads on 1 kv head (head size 32), hidden 160,
     vocabulary 300, rope base 1e6, eps 1e-5, seed 12; both with a separate lm_head;
  3. runs the CLI on a prompt of raw bytes (its merge-less tokenizer maps byte b to token b and
     puts BOS = 256 first) with `--trace`, greedy, 3 new tokens, `--scalar`.
Kept: model.smoe (the Q8 container, ~120 KB), config.ini, prompt.bin, trace.txt (one line per
processed token: position, then the logits as C99 hexadecimal floats), token_ids.txt.

The reference's engine stores weights as Q8 and re-quantizes the input of every matrix product
to Q8 (docs/FORMAT.md), so its logits are those of a slightly different model:
tests/test_golden_reference.py compares statistics (best token, KL), never equality.

    python tests/golden/make_reference_trace.py /path/to/smolmoe-c99
"""
import importlib.util
import os
import shutil
import subprocess
import sys
import tempfile

HERE = os.path.dirname(os.path.abspath(__file__))
FIXTURES = {
    "reference_fixture": (
        dict(architecture="smolmoe_qwen2", dim=64, hidden_dim=128, layers=2, heads=4, kv_heads=2, experts=1, top_k=1,
             vocab_size=258, max_context=128, shared_experts=0, bos_id=256, eos_id=257, rms_eps=1e-6, rope_theta=10000),
        11, bytes([5, 17, 127, 200, 3, 99, 250, 31, 64, 7, 180, 45])),
    "reference_fixture_b": (
        dict(architecture="smolmoe_qwen2", dim=96, hidden_dim=160, layers=3, heads=3, kv_heads=1, experts=1, top_k=1,
             vocab_size=258, max_context=96, shared_experts=0, bos_id=256, eos_id=257, rms_eps=1e-5, rope_theta=1000000),
        12, bytes([(37 * i + 11) % 251 + 1 for i in range(40)])),
}


def main(reference: str) -> None:
    build = os.path.join(tempfile.gettempdir(), "smolmoe_ref_build")
    binary = os.path.join(build, "smolmoe")
    subprocess.run(["make", "-C", reference, f"BUILD={build}", binary], check=True, stdout=subprocess.DEVNULL)
    spec = importlib.util.spec_from_file_location("ref_checkpoint", os.path.join(reference, "tools", "checkpoint.py"))
    checkpoint = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(checkpoint)
    for folder, (config, seed, prompt) in FIXTURES.items():
        out = os.path.join(HERE, folder)
        work = tempfile.mkdtemp(prefix="smolmoe_fixture_")
        checkpoint.fixture(work, config=config, seed=seed)
        with open(os.path.join(work, "prompt.bin"), "wb") as f:
            f.write(prompt)
        env = dict(os.environ, SMOLMOE_KV_CACHE="0")
        subprocess.run([binary, "--model", os.path.join(work, "model.smoe"), "--config", os.path.join(work, "config.ini"),
                        "--tokenizer", os.path.join(work, "tokenizer.bpe"), "--prompt-file", os.path.join(work, "prompt.bin"),
                        "--tokens", "3", "--context", "64", "--scalar", "--threads", "1", "--trace", os.path.join(work, "trace.txt"),
                        "--token-ids", os.path.join(work, "token_ids.txt")], check=True, env=env, stdout=subprocess.DEVNULL,
                       stderr=subprocess.DEVNULL)
        os.makedirs(out, exist_ok=True)
        for name in ("model.smoe", "config.ini", "prompt.bin", "trace.txt", "token_ids.txt"):
            shutil.copyfile(os.path.join(work, name), os.path.join(out, name))
        shutil.rmtree(work)
        print(f"wrote {out}")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_reference_trace.py /path/to/smolmoe-c99")
    main(sys.argv[1])
