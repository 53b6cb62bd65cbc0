"""A GPT as a graph of tensor stages: build the `gpt2_qknorm` preset at toy size, compile it, run a
few training steps with ``TorchTrainer`` on random tokens and print the loss curve. On a B200 the
hot stages run on the sm_100a kernel library; on a CPU box the same graph runs through PyTorch.

    python examples/gpt_graph.py
"""
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))

import torch  # noqa: E402

from neuralfn_b200.presets import build_preset  # noqa: E402
from neuralfn_b200.serialization import graph_to_json  # noqa: E402
from neuralfn_b200.tensor.trainer import TorchTrainConfig, TorchTrainer  # noqa: E402
from neuralfn_b200.torch_templates import build_gpt_root_graph  # noqa: E402


def main() -> int:
    spec = build_preset("gpt2_qknorm", vocab_size=128, num_layers=2, model_dim=64, num_heads=4)
    graph = build_gpt_root_graph(spec)
    print(f"graph: {len(graph.nodes)} nodes, {len(graph_to_json(graph)) // 1024} KiB of JSON")
    device = "cuda" if torch.cuda.is_available() else "cpu"
    cfg = TorchTrainConfig(learning_rate=3e-3, epochs=5, batch_size=8, device=device, seed=0, grad_clip_norm=1.0)
    g = torch.Generator().manual_seed(0)
    tokens = torch.randint(0, 128, (64, 33), generator=g)
    history = TorchTrainer(graph, cfg).train(tokens[:, :-1], tokens[:, 1:])
    print("epoch loss:", " ".join(f"{x:.3f}" for x in history))
    return 0 if history[-1] < history[0] else 1


if __name__ == "__main__":
    raise SystemExit(main())
