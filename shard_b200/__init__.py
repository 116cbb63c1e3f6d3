"""B200-native compressed-KV attention path with the API of bhengubv/shard."""
__all__ = ["Cache", "enable_llama_fused_attention", "fused_attention_compressed"]


def __getattr__(name):
    if name == "Cache":
        from .cache import Cache
        return Cache
    if name in ("enable_llama_fused_attention", "fused_attention_compressed"):
        from . import attention
        return getattr(attention, name)
    raise AttributeError(name)
