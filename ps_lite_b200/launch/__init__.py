"""launch of ps_lite_b200."""
