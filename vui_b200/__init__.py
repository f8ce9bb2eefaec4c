"""vui_b200: Vui Nano's per-codec-frame decode step as sm_100a CUDA behind the
reference's Engine / Row / GenConfig API."""

from .codec import CodecCtx, QwenCodecDecoder
from .engine import Engine, GenConfig, RenderRequest, Row, Segment
from .model import VuiB200, VuiShape

__all__ = ["CodecCtx", "Engine", "GenConfig", "QwenCodecDecoder", "RenderRequest", "Row", "Segment", "VuiB200",
           "VuiShape"]
