"""placeholder, replaced below"""
class Sm100Lowerer:
    pass
ThunderKittensLowerer = Sm100Lowerer
