"""Speculative decoding (draft sources, verify blocks, acceptance)."""
from .decoder import (CopyLookupSource, DraftSource, ModelSource, MtpSource, SamplingState, SpecDecoder,  # noqa: F401
                      SpecStats)
