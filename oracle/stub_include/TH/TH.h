// Stand-in for the PyTorch-0.3 TH umbrella header (nothing from it is used by the kernel files).
