Device = None  # filled in by cupy.cuda.__init__
