"""Bridge for command lines written for llm.c's ``train_gpt2cu``: ``nfn compat-train -- -i ... -o ... -e d12 -b 64 -t 1024``.

The single-letter flags are translated into a ``NativeTrainConfig``; flags that have no meaning
here (recompute, ZeRO stage, sampling cadence, hellaswag, cuDNN switches ...) are accepted and
reported under ``ignored`` so existing launch scripts keep working.

Reference counterpart: ``csrc/native_gpt2/nfn_gpt2_tile_train.cpp`` (the ``-- <train_gpt2cu args>``
compatibility launcher).
"""
from __future__ import annotations

import re

__all__ = ["translate_llmc_args", "LLMC_DEPTHS"]

# "-e dN": depth -> (layers, heads, width), the GPT-2 / GPT-3 ladder llm.c uses
LLMC_DEPTHS = {6: (6, 6, 384), 12: (12, 12, 768), 24: (24, 16, 1024), 36: (36, 20, 1280), 48: (48, 25, 1600)}
_VALUE_FLAGS = {"-i": "train_pattern", "-j": "val_pattern", "-o": "output_dir", "-e": "model", "-b": "batch_size", "-t": "seq_len", "-d": "total_batch",
                "-l": "learning_rate", "-u": "warmup", "-q": "final_lr_frac", "-c": "weight_decay", "-x": "max_steps", "-v": "val_every",
                "-m": "val_batches", "-n": "checkpoint_every", "-y": "resume", "-k": "schedule", "-sl": "outlier_loss", "-sg": "outlier_grad"}
_IGNORED_VALUE_FLAGS = {"-s", "-g", "-h", "-a", "-f", "-w", "-z", "-r", "-nk", "-nm", "-ge", "-lg", "-pn", "-pi", "-pm", "-pf", "-ps"}


def translate_llmc_args(argv: list[str]) -> tuple[dict, dict]:
    """Returns (NativeTrainConfig keyword arguments, {"ignored": {...}}). Unknown flags raise."""
    got, ignored = {}, {}
    it = iter(argv)
    for flag in it:
        if flag in _VALUE_FLAGS or flag in _IGNORED_VALUE_FLAGS:
            try:
                val = next(it)
            except StopIteration:
                raise ValueError(f"flag {flag} needs a value") from None
            (got if flag in _VALUE_FLAGS else ignored)[_VALUE_FLAGS.get(flag, flag)] = val
        else:
            raise ValueError(f"unknown train_gpt2cu flag {flag!r}")
    kw: dict = {"base_model": "gpt", "template_name": "gpt2"}
    if "model" in got:
        m = re.fullmatch(r"d(\d+)", got["model"])
        if not m or int(m.group(1)) not in LLMC_DEPTHS:
            raise ValueError(f"-e wants one of {', '.join('d%d' % d for d in LLMC_DEPTHS)} (checkpoint files are loaded with --resume instead)")
        kw["n_layer"], kw["n_head"], kw["d_model"] = LLMC_DEPTHS[int(m.group(1))]
    if "train_pattern" in got:
        pat = got["train_pattern"]
        kw["dataset"] = pat.rsplit("/", 1)[0] if any(c in pat for c in "*?[") else pat
    for src, dst, conv in (("output_dir", "output_dir", str), ("batch_size", "batch_size", int), ("seq_len", "seq_len", int),
                           ("total_batch", "train_batch_tokens", int), ("learning_rate", "learning_rate", float), ("warmup", "warmup_steps", int),
                           ("final_lr_frac", "final_lr_fraction", float), ("weight_decay", "weight_decay", float), ("max_steps", "max_steps", int),
                           ("val_every", "eval_every", int), ("val_batches", "eval_batches", int), ("checkpoint_every", "checkpoint_every", int)):
        if src in got:
            kw[dst] = conv(got[src])
    if "resume" in got:
        kw["resume"] = got["resume"] not in ("0", "false")
    if "schedule" in got:
        if got["schedule"] not in ("cosine", "constant", "linear", "wsd"):
            raise ValueError("-k wants cosine | constant | linear | wsd")
        kw["lr_schedule"] = "constant" if got["schedule"] == "constant" else "cosine"
        if got["schedule"] in ("linear", "wsd"):
            ignored["-k"] = f"{got['schedule']} (run as cosine)"
    for k in ("val_pattern", "outlier_loss", "outlier_grad"):
        if k in got:
            ignored[k] = got[k]
    return kw, {"ignored": ignored}
