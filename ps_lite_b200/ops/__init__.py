"""ops of ps_lite_b200."""
