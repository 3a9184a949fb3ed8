"""libbarqkv's implementation of the reference's native entry point against the reference's own CUDA
kernel, run side by side on the same seeded inputs: caches and lengths must agree bit for bit.

The reference kernel (``csrc/kernels/paged_kv_cache.cu``) is compiled from a reference checkout by
``oracle/ref_cuda.py`` into ``oracle/_ref``; where that build is absent these tests are skipped (the
same scenarios are still checked against the reference's CPU path through the golden files).
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda"


@pytest.fixture(scope="module")
def reference_kernel():
    from oracle import ref_cuda

    module = ref_cuda.load()
    if module is None:
        pytest.skip("oracle/_ref holds no build of the reference's CUDA kernel")
    return module


@pytest.fixture(scope="module")
def backend():
    from barqtrain_b200 import _ffi

    return _ffi.require_cuda_backend()


def _bits(t):
    return t.contiguous().view(torch.uint8)


@pytest.mark.parametrize("dtype", [torch.float32, torch.float16, torch.bfloat16, torch.float64])
@pytest.mark.parametrize("shape", [
    dict(bmax=3, b=2, h=4, d=64, ps=16, blocks=6, steps=(37, 1, 1, 20, 1, 15, 1)),       # crosses pages mid-append
    dict(bmax=5, b=5, h=2, d=128, ps=4, blocks=9, steps=(2, 2, 1, 4, 5, 1, 3)),          # the reference test's page size
    dict(bmax=2, b=1, h=3, d=40, ps=32, blocks=3, steps=(1, 31, 1, 32, 1)),              # head_dim not a multiple of 32
])
def test_append_matches_the_reference_cuda_kernel(reference_kernel, backend, dtype, shape):
    g = torch.Generator(device=DEV).manual_seed(4321)
    size = (shape["bmax"], shape["h"], shape["blocks"], shape["ps"], shape["d"])
    ref_k, ref_v = torch.zeros(size, dtype=dtype, device=DEV), torch.zeros(size, dtype=dtype, device=DEV)
    our_k, our_v = torch.zeros_like(ref_k), torch.zeros_like(ref_v)
    ref_lens = torch.tensor([3, 0, 7, 1, 2][: shape["bmax"]], dtype=torch.int32, device=DEV)
    our_lens = ref_lens.clone()
    for t in shape["steps"]:
        # [B, T, H, D] storage seen as [B, H, T, D]: the strided view a transformer layer hands over
        k = torch.randn(shape["b"], t, shape["h"], shape["d"], generator=g, device=DEV, dtype=torch.float32).to(dtype)
        v = torch.randn(shape["b"], t, shape["h"], shape["d"], generator=g, device=DEV, dtype=torch.float32).to(dtype)
        k, v = k.transpose(1, 2), v.transpose(1, 2)
        reference_kernel.paged_kv_append_(ref_k, ref_v, ref_lens, k, v)
        backend.paged_kv_append_(our_k, our_v, our_lens, k, v)
        assert torch.equal(our_lens, ref_lens)
        assert torch.equal(_bits(our_k), _bits(ref_k)) and torch.equal(_bits(our_v), _bits(ref_v))
    assert backend.read_status(DEV) == 0


def test_capacity_error_matches_the_reference_cuda_kernel(reference_kernel, backend):
    size = (2, 2, 2, 4, 8)                                   # capacity 8 tokens
    caches = [torch.zeros(size, device=DEV) for _ in range(4)]
    k = torch.ones(2, 2, 3, 8, device=DEV)
    messages = []
    for call, (kc, vc) in ((reference_kernel.paged_kv_append_, caches[:2]), (backend.paged_kv_append_, caches[2:])):
        lens = torch.tensor([2, 6], dtype=torch.int32, device=DEV)
        with pytest.raises(RuntimeError) as err:
            call(kc, vc, lens, k, k)
        messages.append(str(err.value).splitlines()[0])
        assert lens.tolist() == [2, 6] and not bool(kc.any()) and not bool(vc.any())     # all or nothing
    assert "paged KV cache capacity exceeded: requested 9 tokens, max_cache_len=8" in messages[0]
    assert "paged KV cache capacity exceeded: requested 9 tokens, max_cache_len=8" in messages[1]
