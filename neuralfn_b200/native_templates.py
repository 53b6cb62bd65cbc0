"""Template names the native (kernel-library) engines implement, by model family."""
GPT_VARIANTS = ("gpt2", "gpt2_zloss", "gpt2_softcap", "gpt2_qknorm", "gpt2_stable", "gpt2_qknorm_softcap_zloss", "gpt2_diff", "gpt2_moa")
LLAMA_TEMPLATES = ("llama", "llama_fast", "llama_modern", "qwen3_longctx")
NATIVE_FAMILIES = {"gpt": GPT_VARIANTS, "gpt2": GPT_VARIANTS, "gpt3": GPT_VARIANTS, "nanogpt": GPT_VARIANTS, "llama": LLAMA_TEMPLATES}
