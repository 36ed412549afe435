"""Host-side logic that needs no GPU: graph bucket table and dispatch (reference:
vexact/inferencer/cudagraph_utils.py:85-107), pipeline layer split, seeded-noise restatement."""
import pytest
import torch


def test_capture_sizes_are_powers_of_two_up_to_the_first_that_covers_max_size():
    from vexact_b200.cudagraph_utils import CudaGraphManager as M

    assert M.build_capture_sizes(1) == [1]
    assert M.build_capture_sizes(2) == [1, 2]
    assert M.build_capture_sizes(3) == [1, 2, 4]
    assert M.build_capture_sizes(32) == [1, 2, 4, 8, 16, 32]
    assert M.build_capture_sizes(33)[-1] == 64
    for bad in (0, -4, None):
        with pytest.raises(ValueError):
            M.build_capture_sizes(bad)


def _manager(max_tokens, max_seqs, captured=True):
    """A manager with its bucket tables but no CUDA objects: dispatch reads only these."""
    from vexact_b200.cudagraph_utils import BatchExecutionDescriptor as D
    from vexact_b200.cudagraph_utils import CudaGraphManager as M

    m = object.__new__(M)
    m.capture_sizes = M.build_capture_sizes(max_tokens)
    m._descriptors = [D(num_tokens=n, num_seqs=min(n, max_seqs)) for n in m.capture_sizes]
    m._decode_descriptors = [D(num_tokens=n, num_seqs=n, decode=True) for n in m.capture_sizes if n <= max_seqs]
    m.graphs = {d: object() for d in m._descriptors + m._decode_descriptors} if captured else {}
    return m


def test_dispatch_picks_the_smallest_bucket_that_covers_tokens_and_sequences():
    m = _manager(32, 8)
    d = m.dispatch(3, 17, 9)                       # a prefill step: 17 tokens of 3 sequences
    assert (d.num_tokens, d.num_seqs, d.decode) == (32, 8, False)
    d = m.dispatch(3, 3, 1)                        # a decode step: the decode graph of the 4-sequence bucket
    assert (d.num_tokens, d.num_seqs, d.decode) == (4, 4, True)
    d = m.dispatch(1, 1, 1)
    assert (d.num_tokens, d.num_seqs, d.decode) == (1, 1, True)
    d = m.dispatch(8, 8, 1)
    assert (d.num_tokens, d.num_seqs, d.decode) == (8, 8, True)
    d = m.dispatch(2, 6, 5)                        # mixed step, 6 tokens: the 8-token bucket
    assert (d.num_tokens, d.num_seqs, d.decode) == (8, 8, False)
    assert m.dispatch(9, 9, 1) is None             # more sequences than any bucket holds
    assert m.dispatch(2, 33, 32) is None           # more tokens than the largest bucket
    # one token per sequence but not flagged as a decode step: the general graph
    assert m.dispatch(3, 3, None).decode is False


def test_layer_split_matches_the_reference_rule():
    from vexact_b200.inferencer import get_pp_indices

    for layers, pp in [(48, 1), (48, 2), (48, 4), (48, 8), (28, 2), (28, 4), (27, 2), (27, 4), (27, 8), (3, 3)]:
        spans = [get_pp_indices(layers, r, pp) for r in range(pp)]
        assert spans[0][0] == 0 and spans[-1][1] == layers
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))          # contiguous, nothing skipped
        sizes = [b - a for a, b in spans]
        assert max(sizes) - min(sizes) <= 1
    # the splits the 27-layer model gets (reference rule, model_loader.py:141-171)
    assert [b - a for a, b in (get_pp_indices(27, r, 2) for r in range(2))] == [14, 13]
    assert [b - a for a, b in (get_pp_indices(27, r, 4) for r in range(4))] == [7, 7, 7, 6]


def test_seeded_noise_restatement_properties():
    from oracle import sampler as osamp

    q = osamp.seeded_exponential([7, 7, 8], [3, 4, 3], 4099)
    assert q.shape == (3, 4099) and bool((q > 0).all()) and bool(torch.isfinite(q).all())
    assert not torch.equal(q[0], q[1]) and not torch.equal(q[0], q[2])       # position and seed both matter
    assert torch.equal(q[0], osamp.seeded_exponential([7], [3], 4099)[0])    # and nothing else does
    assert torch.equal(q[0, :4096], osamp.seeded_exponential([7], [3], 4096)[0])
    assert abs(float(q.mean()) - 1.0) < 0.05


def test_attention_keys_and_attn_impl_validation():
    """The four `attn_impl` names of the reference (config.py:138) are accepted and registered with HF
    (inferencer.py:51-55); anything else is a ValueError; `flex` refuses CUDA-graph capture elsewhere."""
    from transformers.modeling_utils import ALL_ATTENTION_FUNCTIONS

    from vexact_b200 import attention
    from vexact_b200.config import ModelConfig

    for name in ("fa-invariant", "fa-invariant-cute", "triton-invariant", "flex"):
        assert ModelConfig(attn_impl=name).attn_impl == name
    with pytest.raises(ValueError, match="attn_impl must be one of"):
        ModelConfig(attn_impl="sdpa")
    attention.register_attention_functions()
    for name in ("fa-invariant", "fa-invariant-cute", "triton-invariant"):
        assert ALL_ATTENTION_FUNCTIONS[name] is attention.flash_attention_forward
    assert ALL_ATTENTION_FUNCTIONS["flex"] is attention.flex_attention_forward
