"""B200-native INT4 mixture-of-experts hot path behind the reference's operator boundary."""
