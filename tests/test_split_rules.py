"""The host-side rule that cuts a decode step's contexts into pieces (no GPU needed)."""

from rust_llm_inference_server_b200 import ops


def test_decode_attention_pieces_by_batch_and_context():
    kv = 8
    sms = 148                      # the rule takes the device's count; the numbers below are a B200's
    splits = lambda n, kv, ctx: ops.decode_splits(n, kv, ctx, sms)
    for ctx in (1, 100, 512, 4096, 32768, 131072):
        # from 256 (request, kv head) pairs on the context stays whole
        assert splits(32, kv, ctx) == 1 and splits(200, kv, ctx) == 1
    for n in (1, 2, 4, 8, 12, 16, 24):
        last = 1
        for ctx in (64, 128, 500, 512, 1024, 2048, 4096, 8192, 32768):
            s = splits(n, kv, ctx)
            assert 1 <= s <= 32 and s >= last                    # never fewer pieces for a longer context
            assert s == 1 or ctx // s >= (512 if n * kv >= 64 else 128)    # no piece shorter than that
            if n * kv * min(s, 8) <= 4 * sms and s > 1:
                assert s & (s - 1) == 0                          # merged in a cluster: a power of two
            last = s
    assert splits(8, kv, 4096) == 4 and splits(1, kv, 4096) == 8 and splits(2, kv, 4096) == 8
    assert splits(16, kv, 4096) == 2 and splits(8, kv, 512) == 1
    # the rule is a function of the step's shape only: the same step, the same pieces
    assert splits(3, 2, 7000) == splits(3, 2, 7000)
    # a smaller part fills up with fewer pieces
    assert ops.decode_splits(8, kv, 4096, 32) <= splits(8, kv, 4096)
