"""Per-modality model library: audio, image, vision, video, OCR, text and sentence embeddings (the reference's
engines/trainer/multimodal tree). The fusion models that combine modalities live in ``models.multimodal``."""
from . import api, audio, embeddings, image, ocr, text, video, vision   # noqa: F401
from .audio import MFCC, AudioEncoder, AudioFeatures, MelSpectrogram, SpeechRecognizer   # noqa: F401
from .embeddings import ContrastiveHead, CrossEncoder, DualEncoder, EmbeddingConfig, EmbeddingEncoder, NTXentLoss   # noqa: F401
from .image import ConvBlock, ImageDecoder, ImageEncoder, ImageGenerator, ImageGenResult, ResidualBlock   # noqa: F401
from .ocr import CRNN, AttentionDecoder, GridPositionalEncoding, OCRConfig, TransformerOCR   # noqa: F401
from .text import (BPEEncoder, LearnablePositionalEncoding, PoolingStrategy, SequenceClassifier, SinusoidalPositionalEncoding,   # noqa: F401
                   TextConfig, TextDecoder, TextEncoder)
from .video import (InceptionModule, MotionFeatureExtractor, SplitVideoEncoder, TemporalPositionalEncoding, TemporalTransformer,   # noqa: F401
                    VideoConfig)
from .vision import Conv2dPatchEmbed, LayerNorm2D, VisionEncoder, VisionResult, VisionTask, ViTFeatureExtractor   # noqa: F401
