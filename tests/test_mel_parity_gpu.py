"""logMelWindows (the log-mel front end on the device) against the CPU restatement of the reference's
JsPreprocessor / ParakeetMel.  Floating point: the tolerance is 1e-4 on the normalised features (unit scale)
and on raw log-mel values - both sides run the same algorithm in doubles and differ only in the last bits of
cos/sin/log and in the order of the normalisation sums."""
import numpy as np
import pytest

from oracle.mel_oracle import nemotron_mel, parakeet_mel

pytestmark = pytest.mark.gpu


def _windows(W, n, seed):
    from fluidaudio_web_b200.engines import synth

    return synth.synth_audio(W, samples=n, seed=seed)


@pytest.mark.parametrize("W,n", [(3, 240000), (2, 16000), (1, 163), (4, 1000)])
def test_parakeet_features_match_oracle(ctx, pkg, W, n):
    audio = _windows(W, n, seed=W + n)
    got = ctx.download(ctx.logMelWindows(ctx.upload(audio, W, n))).reshape(W, n // 160, 128)
    for w in range(W):
        ref = parakeet_mel(audio[w])  # [128, T]
        assert np.abs(got[w] - ref.T).max() <= 1e-4


def test_nemotron_raw_log_mel_matches_oracle(ctx, pkg):
    audio = _windows(2, 32000, seed=9)
    got = ctx.download(ctx.logMelWindows(ctx.upload(audio, 2, 32000), 128, 1e-10, False)).reshape(2, 201, 128)
    for w in range(2):
        assert np.abs(got[w] - nemotron_mel(audio[w]).T).max() <= 1e-4


def test_80_mel_bins_and_silence(ctx, pkg):
    audio = _windows(1, 8000, seed=2)
    got = ctx.download(ctx.logMelWindows(ctx.upload(audio, 1, 8000), 80)).reshape(50, 80)
    assert np.abs(got - parakeet_mel(audio[0], 80).T).max() <= 1e-4
    z = ctx.download(ctx.logMelWindows(ctx.upload(np.zeros((1, 4800), np.float32), 1, 4800)))
    assert np.allclose(z, 0.0)


def test_features_feed_the_encoder_front_end(ctx, pkg):
    """The device features are the time-major window image pre_encode_windows reads: same frames as the host path."""
    from fluidaudio_web_b200.engines import fastconformer as fc, synth

    w = synth.encoder_weights(synth.TINY, seed=3)
    enc = fc.load_encoder(ctx, w)
    nm = enc["cfg"]["melBins"]
    audio = _windows(2, 32000, seed=5)
    host_mels = [parakeet_mel(a, nm).reshape(-1) for a in audio]  # channel-major, as ParakeetMel returns them
    h = ctx.pushArena()
    ref, _ = fc.encode_batch(ctx, enc, host_mels)
    want = ctx.download(ref)
    feats = ctx.logMelWindows(ctx.upload(audio, 2, 32000), nm)
    got, _ = fc.encode_batch(ctx, enc, [ctx.sliceRows(feats, i, 1) for i in range(2)])
    assert np.abs(ctx.download(got) - want).max() <= 2e-3
    ctx.popArena(h)
