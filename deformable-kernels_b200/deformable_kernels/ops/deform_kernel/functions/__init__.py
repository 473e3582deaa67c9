from .filter_sample_depthwise import sample_depthwise, deform_sample_depthwise
from .nd_linear_sample import nd_linear_sample
from .plane_scale import plane_scale
from .global_dk import global_dk_scale
from .clip_offsets import clip_offsets

__all__ = ['sample_depthwise', 'deform_sample_depthwise', 'nd_linear_sample', 'plane_scale', 'global_dk_scale', 'clip_offsets']
