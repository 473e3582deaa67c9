from .filter_sample_depthwise import SampleDepthwise, DeformableSampleDepthwise

__all__ = ['SampleDepthwise', 'DeformableSampleDepthwise']
