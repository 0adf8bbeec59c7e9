"""B200-native FlashAttention-2 forward behind the ASCEND-RSFA operator surface."""

__version__ = "0.1.0"
