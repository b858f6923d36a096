"""kernel_agent: discover which NumPy operations trace, compile and run, test generated kernels through
the three stages numpy -> compile -> device, and sweep randomly composed kernels
(counterpart of nkipy/src/nkipy/tools/kernel_agent in the reference)."""
