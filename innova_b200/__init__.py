"""InNova-B200: a Blackwell-native training and inference framework with the capabilities of
origin-labs-ai/InNova (dense and MoE decoders, STE train-in-format quantisation, the .oil container
and its block codecs, fine-tuning on a quantised base, paged-KV inference, speculative decoding)."""
__version__ = "0.1.0"
