"""One small invocation of the hot path on cuda:0, checked against the oracle: the config-1 model, a ragged
prefill step of two prompts and four batched decode steps, logits compared with the reference model's."""

from pathlib import Path

import numpy as np


def run() -> None:
    import torch

    assert torch.cuda.is_available(), "smoke() needs a CUDA device"
    import __graft_entry__ as entry

    entry.load_package()
    from q38b200 import engine as eng

    gold_dir = Path(__file__).resolve().parent / "golden"
    gold = np.load(gold_dir / "tiny_cfg1_golden.npz")
    model = eng.Model(gold_dir / "tiny_cfg1.q38")
    runner = eng.Runner(model, eng.default_runner_options(max_batch=4, prefill_chunk=128, kv_tokens=4096,
                                                          max_context=1024, verbose=0))
    g = eng.greedy()
    prompts = [gold["prompt0"], gold["prompt2"]]
    gens = [gold["gen0"], gold["gen2"]]
    refs = [gold["logits0"].astype(np.float32), gold["logits2"].astype(np.float32)]
    for s in range(2):
        runner.reset_slot(s)
        assert runner.kv_ensure(s, len(prompts[s]) + 8)
    runner.prefill([(0, 0, prompts[0], g, 0), (1, 0, prompts[1], g, 0)])
    worst = 0.0
    for step in range(4):
        runner.decode([(s, len(prompts[s]) + step, int(gens[s][step]), g, step + 1) for s in range(2)])
        logits = runner.last_logits(2)
        for s in range(2):
            want = refs[s][len(prompts[s]) + step]
            worst = max(worst, float(np.abs(logits[s] - want).max() / np.abs(want).max()))
    assert worst <= 2e-2, f"logits differ from the reference model: rel_max {worst}"
    # the oracle restatement itself, on the last step's inputs (checker only)
    from oracle_model import OracleModel

    om = OracleModel(gold_dir / "tiny_cfg1.q38", max_positions=64)
    seq = om.new_sequence()
    full = np.concatenate([prompts[0], gens[0][:4]])
    want = om.forward(seq, full)[-1]
    assert float(np.abs(logits[0] - want).max() / np.abs(want).max()) <= 2e-2
    print(f"smoke ok: rel_max vs reference logits {worst:.3e}")
    runner.close()
    model.close()


if __name__ == "__main__":
    run()
