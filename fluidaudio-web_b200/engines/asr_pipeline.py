"""Windowed transcription batch by batch, samples to token ids, with the stages overlapped the way the reference's
pipeline overlaps them (src/engines/asr-parakeet/pipeline.js:32-61, `pipelined`): while one group of windows is in the
encoder, the group before it is being decoded.  There the decoder runs on CPU workers beside the GPU encoder; here
both are on the GPU, in two contexts (streams): a slot's stream carries its copies, the log-mel front end, the
encoder with the joint's encoder projection riding the same recording, and then the lock-step TDT decode of that
batch, whose short dependent launches run under the long products of the other slot's forward.  Forwards are ordered
against each other on the device (PipelinedEncoder); decodes are not ordered against anything but their own slot.
"""
from __future__ import annotations

from .fastconformer import PipelinedEncoder


class PipelinedAsr(PipelinedEncoder):
    """submit() enqueues the next batch's forward on its slot and then decodes the batch enqueued before it (a host
    call that returns when that decode has finished): it returns the per-window (token ids, emission frames) of the
    batch submitted one call earlier, None on the first call.  flush() decodes what is still pending.

    ctxs, encs: as PipelinedEncoder; decs: TdtDecoder(ctx, weights) per slot; W: windows per batch."""

    def __init__(self, ctxs, encs, decs, host_windows, mel_len: int, W: int, from_pcm: bool = True, resident=None):
        self.decs, self.W = list(decs), W
        super().__init__(ctxs, encs, host_windows, mel_len, from_pcm=from_pcm, resident=resident, read_back=False,
                         post=lambda s, x: self.decs[s].project(x))

    def _decode(self, s):
        proj = self.outs[s]
        return self.decs[s].decode_proj(proj, self.W, proj.rows // self.W)

    def submit(self):
        s = self.next
        self.next = (s + 1) % len(self.ctxs)
        self._launch(s)
        out = self._decode(self.pending.pop(0)) if self.pending else None
        self.pending.append(s)
        return out

    def flush(self):
        res = [self._decode(s) for s in self.pending]
        self.pending = []
        return res
