"""Text-embedding encoder: training lowers both objectives, related texts end up closer, checkpoints
round-trip, and the CLI trains and embeds."""
import json

import torch


def _corpus():
    animals = ["the cat sat on the mat", "a cat sleeps on a mat", "the dog runs in the park", "a dog plays in a park", "birds fly over the lake",
               "a bird flies above a lake"]
    numbers = ["one two three four five", "two three four five six", "seven eight nine ten", "eight nine ten eleven", "twenty thirty forty fifty",
               "thirty forty fifty sixty"]
    return animals + numbers


def test_embedding_training_and_roundtrip(tmp_path):
    from neuralfn_b200.embedding import EmbeddingConfig, EmbeddingEncoder, EmbeddingTrainer, load_embedding_model, save_embedding_model
    torch.manual_seed(0)
    model = EmbeddingEncoder(EmbeddingConfig(hidden_dim=64, output_dim=32, num_layers=2, num_heads=4, max_tokens=48))
    tr = EmbeddingTrainer(model, learning_rate=2e-3, warmup_steps=5, max_steps=60, seed=1)
    hist = tr.train(_corpus(), batch_size=6)
    first, last = sum(h["total"] for h in hist[:5]) / 5, sum(h["total"] for h in hist[-5:]) / 5
    assert len(hist) == 60 and last < first - 0.3, (first, last)
    v = model.embed(["the cat sat on the mat", "the cat sat on the mat!", "thirty forty fifty sixty"])
    assert torch.allclose(v.norm(dim=-1), torch.ones(3), atol=1e-5)
    assert float(v[0] @ v[1]) > float(v[0] @ v[2])
    save_embedding_model(model, tmp_path / "emb", tr)
    again = load_embedding_model(tmp_path / "emb")
    assert torch.allclose(again.embed(["hello world"]), model.embed(["hello world"]), atol=1e-6)
    # padding does not change a text's vector
    alone, padded = model.embed(["short"]), model.embed(["short", "a much longer text that forces padding of the first one"])
    assert torch.allclose(alone[0], padded[0], atol=1e-5)


def test_embedding_cli(tmp_path, capsys):
    from neuralfn_b200.cli import nfn
    data = tmp_path / "corpus.txt"
    data.write_text("\n".join(_corpus()))
    rc = nfn.main(["train", "--base-model", "embedding", "--embedding-dataset", str(data), "--embedding-hidden-dim", "32", "--embedding-output-dim", "16",
                   "--embedding-layers", "1", "--embedding-heads", "2", "--embedding-max-tokens", "32", "--batch-size", "4", "--max-steps", "6",
                   "--progress-every", "2", "--output-dir", str(tmp_path / "out")])
    lines = [json.loads(l) for l in capsys.readouterr().out.splitlines() if l.startswith("{")]
    assert rc == 0 and lines[-1]["event"] == "complete" and lines[-1]["steps"] == 6 and sum(l["event"] == "train_step" for l in lines) == 3
    assert nfn.main(["embed", "--checkpoint", str(tmp_path / "out"), "--text", "the cat"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["dim"] == 16 and abs(sum(x * x for x in out["embeddings"][0]) - 1.0) < 1e-3
