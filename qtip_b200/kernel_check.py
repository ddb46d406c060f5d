"""Which configurations the fused HYB kernel covers (lib/utils/kernel_check.py:1-14 upstream)."""


def has_kernel(decode_mode, L, K, V, tlut_bits, td_x, td_y):
    return (decode_mode == 'quantlut_sym' and L == 16 and V == 2 and 2 <= K <= 4 and tlut_bits == 9
            and td_x == 16 and td_y == 16)
