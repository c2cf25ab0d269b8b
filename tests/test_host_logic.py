"""Host-side rules that need no GPU: the decode split-size rule and its environment override, the padded
capacity of moe_align_block_size."""


def test_decode_split_size_rule(monkeypatch):
    from dlcompiler_b200.kernels import paged_attention as pa

    monkeypatch.delenv("DLBLAS_B200_DECODE_CHUNK", raising=False)
    # C5: 64 sequences x 8 kv heads x up to 32768 tokens -> the longest split the rule allows
    assert pa._pick_chunk(64, 8, 32768, 64) == 4096
    # 16 sequences: about 4 waves of CTAs
    assert pa._pick_chunk(16, 8, 32768, 64) == 2048
    # tiny problems: never below one 256-token split, never below a page
    assert pa._pick_chunk(1, 1, 100, 16) == 256
    assert pa._pick_chunk(1, 1, 100, 1024) == 1024
    for b, h, c, p in [(3, 2, 5000, 32), (128, 8, 2048, 16), (7, 1, 70000, 128)]:
        chunk = pa._pick_chunk(b, h, c, p)
        assert chunk & (chunk - 1) == 0 and chunk % 64 == 0 and chunk % min(p, chunk) == 0
    monkeypatch.setenv("DLBLAS_B200_DECODE_CHUNK", "300")
    assert pa._pick_chunk(64, 8, 32768, 64) == 512          # rounded up to a power of two
    monkeypatch.setenv("DLBLAS_B200_DECODE_CHUNK", "64")
    assert pa._pick_chunk(64, 8, 32768, 256) == 256         # never below a page


def test_align_capacity_covers_the_worst_case():
    from dlcompiler_b200.kernels.fused_moe import _align_capacity

    for numel, experts, block in [(8192, 8, 128), (1, 4, 128), (0, 3, 16), (1000, 256, 64), (77, 7, 1)]:
        cap = _align_capacity(numel, experts, block)
        assert cap % block == 0
        assert cap >= numel + experts * (block - 1)          # every expert may waste block - 1 entries
        assert cap - (numel + experts * (block - 1)) < block

