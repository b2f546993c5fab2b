"""Host-side bookkeeping of the synthetic dense decoder (no GPU)."""


def test_packed_byte_count():
    from ponyexl3_b200.dense_step import DenseConfig, draw_bit_widths
    cfg = DenseConfig()
    ks = draw_bit_widths(cfg, 5000)
    total = cfg.packed_bytes(ks)
    # 21.9 G weights at 4..5 bits: between 4.0 and 4.4 bits per weight on average
    weights = cfg.layers * 330_301_440 + cfg.hidden * cfg.vocab
    assert 4.0 <= 8 * total / weights <= 4.4
