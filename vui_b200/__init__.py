"""vui_b200: Vui Nano's per-codec-frame decode step as sm_100a CUDA behind the
reference's Engine / Row / GenConfig API."""

from .codec import CodecCtx, QwenCodecDecoder
from .codec_encoder import QwenCodecEncoder, StreamingCodecEncoder
from .engine import Engine, GenConfig, RenderRequest, Row, Segment
from .model import VuiB200, VuiShape

__all__ = ["CodecCtx", "Engine", "GenConfig", "QwenCodecDecoder", "QwenCodecEncoder", "RenderRequest", "Row", "Segment",
           "StreamingCodecEncoder", "VuiB200", "VuiShape"]
