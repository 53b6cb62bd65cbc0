"""Weight quantisation formats: GGUF K-quants (Q4_K/Q5_K/Q6_K), NF4, TurboQuant KV."""
from . import kquant

__all__ = ["kquant"]
