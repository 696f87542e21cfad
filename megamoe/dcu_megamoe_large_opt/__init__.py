"""Import path of the reference's staged-path helpers (megamoe/dcu_megamoe_large_opt/), served by the B200 library."""
