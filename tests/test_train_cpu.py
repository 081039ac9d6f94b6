"""Host-side pieces of the trainer that need no GPU: HellaSwag scoring on a small JSONL file,
the held-out validation split of a token file, per-rank loader state in checkpoints."""
import json
import socket

import pytest
import torch

from zero_to_hero_b200.config import get_preset
from zero_to_hero_b200.data.synthetic import SyntheticLoader
from zero_to_hero_b200.data.text import TokenFileLoader
from zero_to_hero_b200.engine import select_rank_state
from zero_to_hero_b200.eval.hellaswag import evaluate, evaluate_losses_fn, load_examples
from zero_to_hero_b200.models.gpt2 import GPT2


def _examples():
    g = torch.Generator().manual_seed(0)
    out = []
    for i in range(3):
        ctx = torch.randint(0, 500, (12 + i,), generator=g).tolist()
        ends = [torch.randint(0, 500, (4 + j,), generator=g).tolist() for j in range(4)]
        out.append({"ctx_tokens": ctx, "ending_tokens": ends, "label": i})
    return out


def test_hellaswag_scoring_on_three_examples(tmp_path):
    """Both scoring routes (logits, per-token losses) agree with a direct restatement of the
    reference's rule (nn/gpt2/hellaswag.py:41-60): mean loss over the ending's tokens, argmin."""
    path = tmp_path / "hs.jsonl"
    path.write_text("\n".join(json.dumps(e) for e in _examples()) + "\n")
    examples = load_examples(path)
    assert len(examples) == 3
    cfg = get_preset("gpt2-tiny")
    cfg.model.block_size = 256
    torch.manual_seed(0)
    model = GPT2(cfg.model).eval()

    def losses_fn(t, tgt):
        with torch.no_grad():
            logits, _ = model(t, tgt)
        return torch.nn.functional.cross_entropy(logits.view(-1, logits.size(-1)), tgt.view(-1),
                                                 reduction="none").view(t.shape)

    c1, n1 = evaluate(model, examples, "cpu", 256)
    c2, n2 = evaluate_losses_fn(losses_fn, examples, "cpu", 256)
    assert int(n1) == int(n2) == 3 and int(c1) == int(c2)
    # direct restatement for every example
    correct = 0
    for ex in examples:
        best, best_loss = -1, float("inf")
        for j, end in enumerate(ex["ending_tokens"]):
            toks = torch.tensor(ex["ctx_tokens"] + end)[None]
            with torch.no_grad():
                logits, _ = model(toks, toks)
            ce = torch.nn.functional.cross_entropy(logits[0, :-1], toks[0, 1:], reduction="none")
            loss = ce[-len(end):].mean().item()
            if loss < best_loss:
                best, best_loss = j, loss
        correct += int(best == ex["label"])
    assert correct == int(c1)
    # strided over two ranks, summed: the two all-reduces of the trainer add exactly these
    parts = [evaluate(model, examples, "cpu", 256, r, 2) for r in range(2)]
    assert sum(int(n) for _, n in parts) == 3 and sum(int(c) for c, _ in parts) == int(c1)


def test_token_file_validation_split_is_held_out_and_unsharded(tmp_path):
    path = tmp_path / "tok.bin"
    import numpy as np
    np.arange(40_000, dtype=np.uint16).tofile(path)
    tr0 = TokenFileLoader(path, 2, 64, rank=0, world_size=2, split="train", val_frac=0.1)
    tr1 = TokenFileLoader(path, 2, 64, rank=1, world_size=2, split="train", val_frac=0.1)
    va = TokenFileLoader(path, 2, 64, rank=0, world_size=1, split="val", val_frac=0.1)
    assert len(va.tokens) == 4000 and int(va.tokens[0]) == 36_000
    assert int(tr0.tokens.max()) < 36_000          # training never sees the tail
    x0, _ = tr0.next_host_batch()
    x1, _ = tr1.next_host_batch()
    assert int(x0[0, 0]) == 0 and int(x1[0, 0]) == 128   # rank shards are disjoint
    xv, yv = va.next_host_batch()
    assert int(xv[0, 0]) == 36_000 and int(yv[0, 0]) == 36_001
    before = tr0.cursor
    va.next_host_batch()
    assert tr0.cursor == before                     # evaluating does not move the training cursor


def test_per_rank_loader_states_round_trip():
    """A 2-rank job's data states are stored per rank and handed back per rank, so that after a
    resume the ranks go on with DIFFERENT batches (each its own stream), not rank 0's."""
    loaders = [SyntheticLoader("train", 2, 16, 100, "cpu", r, 2, seed=7) for r in range(2)]
    for ld in loaders:
        ld.next_host_batch()
    saved = {"world": 2, "per_rank": [ld.state() for ld in loaders]}
    want = [ld.next_host_batch()[0] for ld in loaders]
    fresh = [SyntheticLoader("train", 2, 16, 100, "cpu", r, 2, seed=7) for r in range(2)]
    for r, ld in enumerate(fresh):
        ld.load_state(select_rank_state(saved, r, 2))
    got = [ld.next_host_batch()[0] for ld in fresh]
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
    assert not torch.equal(got[0], got[1])
    with pytest.raises(ValueError):
        select_rank_state(saved, 0, 3)


def test_elastic_resume_reshards_the_token_stream(tmp_path):
    """A checkpoint of a 4-rank job resumed by 2 ranks (and by 8): with `elastic` the token-file
    loaders carry on where the old job's stream stood, each new rank on its own stride, so nothing
    already consumed is read again and nothing is skipped."""
    import numpy as np
    from zero_to_hero_b200.data.text import TokenFileLoader
    path = tmp_path / "tokens.bin"
    np.arange(40000, dtype=np.uint16).tofile(path)  # token value == position in the file
    B, T = 2, 16
    span = B * T
    old = [TokenFileLoader(path, B, T, rank=r, world_size=4) for r in range(4)]
    for _ in range(3):
        for ld in old:
            ld.next_host_batch()
    consumed = 3 * 4 * span
    saved = {"world": 4, "per_rank": [ld.state() for ld in old]}
    for new_world in (2, 8):
        new = [TokenFileLoader(path, B, T, rank=r, world_size=new_world) for r in range(new_world)]
        for r, ld in enumerate(new):
            ld.load_state(select_rank_state(saved, r, new_world, elastic=True))
        firsts = [int(ld.next_host_batch()[0][0, 0]) for ld in new]
        assert firsts == [consumed + r * span for r in range(new_world)]
        seconds = [int(ld.next_host_batch()[0][0, 0]) for ld in new]
        assert seconds == [consumed + (new_world + r) * span for r in range(new_world)]
    # the synthetic loader: surviving ranks keep their generators, so their streams continue
    syn = [SyntheticLoader("train", 2, 16, 100, "cpu", r, 4, seed=7) for r in range(4)]
    for ld in syn:
        ld.next_host_batch()
    saved = {"world": 4, "per_rank": [ld.state() for ld in syn]}
    want = [ld.next_host_batch()[0] for ld in syn[:2]]
    fresh = [SyntheticLoader("train", 2, 16, 100, "cpu", r, 2, seed=7) for r in range(2)]
    for r, ld in enumerate(fresh):
        ld.load_state(select_rank_state(saved, r, 2, elastic=True))
    got = [ld.next_host_batch()[0] for ld in fresh]
    assert torch.equal(got[0], want[0]) and torch.equal(got[1], want[1])
