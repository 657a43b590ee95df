"""gmc: Gaussian-mixture operators for Gaussian Mixture Convolution Networks on B200 (sm_100a).

Mirrors the operator surface of the reference's src/gmc package (mixture packing, evaluation,
integration, fitting, convolution) on top of libgmc_b200.so.
"""
